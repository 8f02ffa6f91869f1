/*
 * vyre_b200.h - C ABI of libvyre_b200.so: a Blackwell (sm_100a) native backend for vyre's
 * quantized-inference hot path (weight-only quantized linear + MoE expert dispatch).
 *
 * The reference boundary is a set of Rust traits plus an `inventory` registration; it has no C ABI.
 * Every export below flattens exactly one reference item (cited as file:line within the vyre tree), so
 * that a small Rust shim inside vyre-driver-cuda (`impl TargetCompiler`, `impl ArtifactMaterializer`,
 * `impl ArtifactInstance`, `impl Submission`) forwards each trait method to one function here.
 *
 * Conventions
 *  - every function returns an int32 status: 0 = ok, otherwise the reference's stable error id
 *    (vyre-driver/src/backend/error.rs:47-59); the message of the last failure on the calling thread is
 *    available from vyb_last_error_message() and always contains "Fix: ".
 *  - nothing panics, traps or falls back to the CPU: a missing or non-sm_100 device is a structured
 *    failure (vyre README.md:36-37).
 *  - all pointers are plain host pointers unless a parameter is documented as a device pointer.
 *  - handles are opaque and thread-safe; `*_free` accepts NULL.
 */
#ifndef VYRE_B200_H
#define VYRE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VYB_ABI_VERSION 1u

/* ---- error ids: vyre-driver/src/backend/error.rs:47-59 (ErrorCode::stable_id) -------------------- */
#define VYB_OK 0
#define VYB_ERR_DEVICE_OUT_OF_MEMORY 1001
#define VYB_ERR_UNSUPPORTED_FEATURE 1002
#define VYB_ERR_POISONED_LOCK 1003
#define VYB_ERR_KERNEL_COMPILE_FAILED 1004
#define VYB_ERR_DISPATCH_FAILED 1005
#define VYB_ERR_INVALID_PROGRAM 1006
#define VYB_ERR_COOPERATIVE_RESIDENCY_EXCEEDED 1007
#define VYB_ERR_DEVICE_LOST 1008
#define VYB_ERR_UNKNOWN 1999
/* DispatchError of the self-substrate wrappers (vyre-self-substrate/src/optimizer/dispatcher.rs:100-120): Rejected,
 * BadInputs, BackendError; the message carries the reference's Display prefix */
#define VYB_ERR_DISPATCH_REJECTED 2001
#define VYB_ERR_DISPATCH_BAD_INPUTS 2002
#define VYB_ERR_DISPATCH_BACKEND 2003

/* ---- DataType tags: vyre-spec/src/data_type.rs:2-8,227-257 ---------------------------------------- */
#define VYB_DT_U32 0x01u
#define VYB_DT_I32 0x02u
#define VYB_DT_F16 0x09u
#define VYB_DT_BF16 0x0Au
#define VYB_DT_F32 0x0Bu
#define VYB_DT_U8 0x0Eu
#define VYB_DT_I8 0x10u
#define VYB_DT_I4 0x1Bu
#define VYB_DT_QUANTIZED 0x1Fu

/* BufferAccess: vyre-foundation/src/ir_inner/model/program/buffer_decl.rs */
#define VYB_ACCESS_READ_ONLY 0u
#define VYB_ACCESS_READ_WRITE 1u
#define VYB_ACCESS_OUTPUT 2u    /* backend-allocated, zero-initialised output */
#define VYB_ACCESS_WORKGROUP 3u /* workgroup scratch, never bound */

typedef struct vyb_program vyb_program;       /* vyre_foundation::ir::Program */
typedef struct vyb_artifact vyb_artifact;     /* vyre_megakernel::Artifact */
typedef struct vyb_payload vyb_payload;       /* vyre_megakernel::TargetPayload */
typedef struct vyb_device vyb_device;         /* vyre_driver Device + ArtifactMaterializer */
typedef struct vyb_instance vyb_instance;     /* vyre_driver ArtifactInstance */
typedef struct vyb_submission vyb_submission; /* vyre_driver Submission */
typedef struct vyb_prepared vyb_prepared;     /* a BindingSet frozen for replay (no counterpart in the reference) */
typedef struct vyb_completion vyb_completion; /* vyre_driver Completion */

/* vyre-driver/src/backend/resource.rs:22-84 (ResidentHandle = owner + id) */
typedef struct vyb_resident_handle {
    uint64_t owner;
    uint64_t id;
} vyb_resident_handle;

/* vyre-megakernel TargetProfile as used by CudaTargetCompiler (vyre-driver-cuda/src/target_compiler.rs:35-71) */
typedef struct vyb_target_profile {
    char identity[64];
    uint32_t generation; /* 100 = sm_100a */
    uint32_t max_workgroup_size[3];
    uint32_t max_invocations;
    uint32_t max_dynamic_shared_bytes;
    uint32_t subgroup_size;
} vyb_target_profile;

/* BackendRegistration: vyre-driver/src/backend/registry/inventory_streams.rs:38-69 */
typedef struct vyb_registration_info {
    const char* id;             /* "cuda-b200" */
    const char* target_id;      /* "nvidia-sm100a" */
    const char* payload_format; /* "b200-native" */
    uint32_t format_version;    /* 1 */
    uint32_t precedence;        /* rank among backends, CUDA's own is 5 (vyre-driver-cuda/src/lib.rs:1083-1088) */
    vyb_target_profile profile;
} vyb_registration_info;

/* DeviceIdentity: vyre-driver/src/backend/artifact_lifecycle.rs:11-19 */
typedef struct vyb_device_identity {
    char backend[32];
    char device[96];
    uint64_t generation;
} vyb_device_identity;

/* CudaDeviceCaps subset: vyre-driver-cuda/src/device.rs:40-85 */
typedef struct vyb_device_caps {
    char name[128];
    int32_t ordinal;
    int32_t compute_major, compute_minor;
    uint64_t total_memory;
    int32_t max_threads_per_block;
    int32_t shared_memory_per_block, shared_memory_per_sm, shared_memory_per_block_optin;
    int32_t warp_size;
    int32_t cooperative_launch;
    int32_t multi_processor_count;
    int32_t l2_cache_bytes;
    int32_t memory_clock_rate_khz, core_clock_rate_khz, global_memory_bus_width_bits;
} vyb_device_caps;

/* BufferDecl view: vyre-foundation/src/ir_inner/model/program/buffer_decl.rs */
typedef struct vyb_buffer_decl {
    const char* name; /* owned by the program */
    uint32_t binding;
    uint32_t access;
    uint32_t dtype;
    uint32_t count;                 /* elements */
    uint32_t has_output_byte_range; /* with_output_byte_range (linear_4bit.rs:743-771) */
    uint64_t output_byte_begin, output_byte_end;
} vyb_buffer_decl;

/* QuantizedLinear4BitSpec: vyre-libs/src/nn/linear/inner/linear_4bit.rs:78-134 */
typedef struct vyb_quantized_linear_4bit_spec {
    uint32_t in_dim, out_dim;
    uint32_t storage_dtype;        /* VYB_DT_I4 for a valid spec */
    uint32_t scale_group_size;     /* QuantizationScale::PerGroup */
    uint32_t zero_point_group_size; /* QuantizationZeroPoint::PerGroup */
} vyb_quantized_linear_4bit_spec;

/* QuantizedLinear4BitPlannerEvidence: linear_4bit.rs:30-69 */
typedef struct vyb_planner_evidence {
    uint32_t in_dim, out_dim, group_size, group_count;
    uint64_t packed_weight_bytes, dequantized_weight_bytes, sidecar_bytes, bias_bytes, output_bytes;
    uint64_t dequant_bytes_elided;
    uint32_t matmul_m, matmul_k, matmul_n, matmul_tile;
    const char* matmul_selected_path;
    const char* matmul_candidate_path;  /* NULL when none */
    const char* matmul_fallback_reason; /* NULL when none */
    uint32_t tensor_core_eligible;
    float output_drift_abs_tolerance; /* LINEAR_4BIT_AFFINE_GROUPED_OUTPUT_DRIFT_ABS_TOLERANCE = 1e-4 */
} vyb_planner_evidence;

/* BoundResource: vyre-driver/src/backend/artifact_lifecycle.rs:32-39 */
#define VYB_BIND_HOST 0
#define VYB_BIND_RESIDENT 1
typedef struct vyb_binding {
    uint32_t value_id; /* ArtifactValueId = BufferDecl binding slot */
    int32_t kind;
    const void* host_ptr; /* VYB_BIND_HOST: bytes are copied in during vyb_submit */
    size_t len;
    vyb_resident_handle resident; /* VYB_BIND_RESIDENT */
} vyb_binding;

/* DispatchConfig: vyre-driver/src/backend/dispatch_config.rs:26-110. Only grid, timeout_ns, label and
 * leave_resident are honoured; a non-zero value in any other field is refused with UnsupportedFeature. */
typedef struct vyb_dispatch_config {
    uint32_t grid_override[3]; /* all zero = none; a zero axis next to non-zero ones is InvalidProgram */
    uint32_t workgroup_override[3];
    uint64_t timeout_ns;
    const char* label;
    uint32_t ulp_budget;
    uint64_t max_output_bytes;
    uint32_t cooperative;
    uint32_t leave_resident; /* 1: outputs written into caller-bound resident buffers are not read back */
} vyb_dispatch_config;

/* ---- library ---------------------------------------------------------------------------------- */
uint32_t vyb_abi_version(void);
/* thread-local text of the last failure; BackendError Display (error.rs:83-191) */
const char* vyb_last_error_message(void);
/* BackendRegistration static (inventory_streams.rs:38-69; CUDA's instance vyre-driver-cuda/src/lib.rs:1068-1080) */
int32_t vyb_registration(vyb_registration_info* out);
/* BackendRegistration::supported_ops */
uint32_t vyb_supported_op_count(void);
const char* vyb_supported_op(uint32_t index);
/* blake3 (the digest of Artifact/TargetPayload identities, vyre-megakernel/src/lib.rs:52-59) */
void vyb_blake3(const void* data, size_t len, uint8_t out[32]);

/* ---- operator surface: vyre-libs::nn::{linear,quant,moe,activation}; vyre-primitives::math::quantized -- */
/* Same argument order as the Rust builders: buffer names, then dimensions. A builder that returns
 * Result<Program,String> in the reference returns InvalidProgram with the same "Fix: ..." text here; a
 * builder that returns a trap Program in the reference returns a program with vyb_program_is_trap() = 1. */

/* linear_4bit.rs:255 */
int32_t vyb_nn_linear_4bit(const char* x, const char* w_packed, const char* b, const char* out, uint32_t in_dim,
                           uint32_t out_dim, vyb_program** program);
/* linear_4bit.rs:357 */
int32_t vyb_nn_linear_4bit_affine_grouped(const char* x, const char* w_packed, const char* scale,
                                          const char* zero_point, const char* b, const char* out, uint32_t in_dim,
                                          uint32_t out_dim, uint32_t group_size, vyb_program** program);
/* linear_4bit.rs:382 */
int32_t vyb_nn_linear_4bit_affine_grouped_batched(const char* x, const char* w_packed, const char* scale,
                                                  const char* zero_point, const char* b, const char* out,
                                                  uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                                  uint32_t batch_size, vyb_program** program);
/* QuantizedLinear4BitSpec::affine_grouped, linear_4bit.rs:90 */
void vyb_quantized_linear_4bit_spec_affine_grouped(uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                                   vyb_quantized_linear_4bit_spec* spec);
/* linear_4bit.rs:1004 */
int32_t vyb_nn_linear_4bit_affine_grouped_typed(const vyb_quantized_linear_4bit_spec* spec, const char* x,
                                                const char* w_packed, const char* scale, const char* zero_point,
                                                const char* b, const char* out, vyb_program** program);
/* linear_4bit.rs:1033 */
int32_t vyb_nn_linear_4bit_affine_grouped_batched_typed(const vyb_quantized_linear_4bit_spec* spec,
                                                        uint32_t batch_size, const char* x, const char* w_packed,
                                                        const char* scale, const char* zero_point, const char* b,
                                                        const char* out, vyb_program** program);
/* linear_4bit.rs:140 */
int32_t vyb_nn_linear_4bit_affine_grouped_planner_evidence(const vyb_quantized_linear_4bit_spec* spec,
                                                           vyb_planner_evidence* out);

/* vyre-primitives/src/math/quantized/programs.rs:21,86,129,186,243,309,457. `lib_op_id` != 0 tags the
 * program with the vyre-libs::quant::int4_* id of the library wrapper (vyre-libs/src/nn/quant/int4.rs:34-40,
 * 110-195) instead of the primitive id. */
int32_t vyb_math_unpack_i4x8(const char* packed_words, const char* out_lanes, uint32_t lane_count,
                             vyb_program** program);
int32_t vyb_math_i4x8_dot_i32(const char* lhs, const char* rhs, const char* out, uint32_t lane_count,
                              uint32_t lib_op_id, vyb_program** program);
int32_t vyb_math_i4x8_dot_f32_scaled(const char* lhs, const char* rhs, const char* lhs_scale, const char* rhs_scale,
                                     const char* out, uint32_t lane_count, uint32_t lib_op_id,
                                     vyb_program** program);
int32_t vyb_math_i4x8_matvec_f32_scaled(const char* weights, const char* x, const char* row_scales, const char* out,
                                        uint32_t rows, uint32_t cols, uint32_t lib_op_id, vyb_program** program);
int32_t vyb_math_i4x8_batched_matvec_f32_scaled(const char* weights, const char* x, const char* row_scales,
                                                const char* out, uint32_t batch, uint32_t rows, uint32_t cols,
                                                uint32_t lib_op_id, vyb_program** program);
int32_t vyb_math_i4x8_batched_matmul_f32_scaled(const char* weights, const char* activations,
                                                const char* row_scales, const char* batch_scales, const char* out,
                                                uint32_t batch, uint32_t rows, uint32_t cols, uint32_t lib_op_id,
                                                vyb_program** program);
int32_t vyb_math_i4x8_batched_matmul_top1_f32_scaled(const char* weights, const char* activations,
                                                     const char* row_scales, const char* batch_scales,
                                                     const char* out_scores, uint32_t batch, uint32_t rows,
                                                     uint32_t cols, uint32_t lib_op_id, vyb_program** program);
/* i4_packed_words, vyre-primitives/src/math/quantized.rs:58-60 */
uint32_t vyb_i4_packed_words(uint32_t lane_count);

/* vyre-libs/src/nn/quant/int8.rs:15,54 */
int32_t vyb_quant_int8_unpack(const char* packed, const char* scales, const char* output, uint32_t n, uint32_t cols,
                              vyb_program** program);
int32_t vyb_quant_int8_pack(const char* input, const char* output, uint32_t n, vyb_program** program);

/* vyre-libs/src/nn/linear/inner/builder.rs:172,202,220,241 (dtype: VYB_DT_F16 / BF16 / F32) */
int32_t vyb_nn_linear_rows(const char* x, const char* w, const char* b, const char* out, uint32_t rows,
                           uint32_t in_dim, uint32_t out_dim, vyb_program** program);
int32_t vyb_nn_linear_rows_no_bias(const char* x, const char* w, const char* out, uint32_t rows, uint32_t in_dim,
                                   uint32_t out_dim, vyb_program** program);
int32_t vyb_nn_linear_rows_no_bias_typed(const char* x, const char* w, const char* out, uint32_t rows,
                                         uint32_t in_dim, uint32_t out_dim, uint32_t dtype, vyb_program** program);
int32_t vyb_nn_linear_rows_no_bias_out_in_typed(const char* x, const char* w, const char* out, uint32_t rows,
                                                uint32_t in_dim, uint32_t out_dim, uint32_t dtype,
                                                vyb_program** program);
/* vyre-libs/src/math/linalg/matmul.rs:17-60 (wrapping u32) */
int32_t vyb_math_matmul(const char* a, const char* b, const char* out, uint32_t m, uint32_t k, uint32_t n,
                        vyb_program** program);
/* vyre-libs/src/math/linalg/matmul.rs:138-271 (MatmulBias: out[i, j] = sum_k a[i, k] * b[k, j] + bias[j], wrapping u32;
 * buffers a=0, b=1, bias=2, out=3) and matmul_tiled/ops.rs:261-337 + program.rs:105-200 (the tiled form declares two
 * workgroup tiles and an output padded to 16 x 16 tiles with the logical bytes as its readback range) */
int32_t vyb_math_matmul_bias(const char* a, const char* b, const char* bias, const char* out, uint32_t m, uint32_t k,
                             uint32_t n, vyb_program** program);
int32_t vyb_math_matmul_bias_tiled(const char* a, const char* b, const char* bias, const char* out, uint32_t m, uint32_t k,
                                   uint32_t n, uint32_t tile, vyb_program** program);
/* vyre-libs/src/nn/linear/inner/builder.rs:139-162 (nn::linear: out[i] = sum_k x[k] * w[k, i] + b[i] over MatmulBias with
 * m = 1; hands over to linear_tiled with tile 32 from in_dim * out_dim >= 1024) and tiled.rs:13-50 (nn::linear_tiled) */
int32_t vyb_nn_linear(const char* x, const char* w, const char* b, const char* out, uint32_t in_dim, uint32_t out_dim,
                      vyb_program** program);
int32_t vyb_nn_linear_tiled(const char* x, const char* w, const char* b, const char* out, uint32_t in_dim, uint32_t out_dim,
                            uint32_t tile, vyb_program** program);

/* vyre-libs/src/nn/moe/gating.rs:19; softmax_top_k.rs:25; top_k.rs:18 */
int32_t vyb_nn_moe_gate(const char* input_scores, const char* output_indices, const char* output_weights,
                        uint32_t num_experts, uint32_t k, vyb_program** program);
int32_t vyb_nn_softmax_top_k(const char* scores, const char* out_indices, const char* out_weights, uint32_t n,
                             uint32_t k, vyb_program** program);
int32_t vyb_nn_top_k(const char* input, const char* output_indices, uint32_t n, uint32_t k, vyb_program** program);
/* vyre-libs/src/nn/activation/swiglu.rs:17,26 */
int32_t vyb_nn_swiglu(const char* gate, const char* up, const char* output, uint32_t n, vyb_program** program);
int32_t vyb_nn_swiglu_typed(const char* gate, const char* up, const char* output, uint32_t n, uint32_t dtype,
                            vyb_program** program);
/* residual_add / residual_add_typed: vyre-libs/src/nn/activation/residual_add.rs:8-52 (out = cast(f32 sum)) */
int32_t vyb_nn_residual_add(const char* residual, const char* branch, const char* output, uint32_t n, vyb_program** program);
int32_t vyb_nn_residual_add_typed(const char* residual, const char* branch, const char* output, uint32_t n, uint32_t dtype,
                                  vyb_program** program);
/* learned_rms_norm / gated_rms_norm: vyre-libs/src/nn/norm/gated_rms_norm.rs:35-247 (f32 sum of squares in row order,
 * 1 / sqrt(mean + eps), rounding to dtype, learned scale, optional SiLU gate, one final cast) */
int32_t vyb_nn_learned_rms_norm(const char* input, const char* weight, const char* output, uint32_t rows, uint32_t hidden,
                                float eps, uint32_t dtype, vyb_program** program);
int32_t vyb_nn_gated_rms_norm(const char* input, const char* weight, const char* gate, const char* output, uint32_t rows,
                              uint32_t hidden, float eps, uint32_t dtype, vyb_program** program);
/* gated_rms_norm_with_weight_dtype (gated_rms_norm.rs:67-96): the learned scale stored in a floating type of its own
 * (bf16 activations with f32 scales, as checkpoints hold them) */
int32_t vyb_nn_gated_rms_norm_with_weight_dtype(const char* input, const char* weight, const char* gate, const char* output,
                                                uint32_t rows, uint32_t hidden, float eps, uint32_t dtype, uint32_t weight_dtype,
                                                vyb_program** program);
/* GGML K-quants with per-block f32 scale / min sidecars: vyre-libs/src/nn/quant/ggml.rs:28-120 (unpack), 217-400 (fused
 * dequant + linear over the k-major weight stream, out = x @ dequant(w) + b) */
int32_t vyb_quant_q4_k_unpack(const char* packed, const char* scales, const char* mins, const char* output, uint32_t n,
                              vyb_program** program);
int32_t vyb_quant_q2_k_unpack(const char* packed, const char* scales, const char* mins, const char* output, uint32_t n,
                              vyb_program** program);
int32_t vyb_quant_q4_k_linear(const char* x, const char* w_packed, const char* w_scales, const char* w_mins, const char* b,
                              const char* out, uint32_t in_dim, uint32_t out_dim, vyb_program** program);
int32_t vyb_quant_q2_k_linear(const char* x, const char* w_packed, const char* w_scales, const char* w_mins, const char* b,
                              const char* out, uint32_t in_dim, uint32_t out_dim, vyb_program** program);
/* vyre-libs/src/nn/moe/expert_mlp.rs:18 */
int32_t vyb_nn_expert_mlp(const char* x, const char* w_gate, const char* b_gate, const char* w_up, const char* b_up,
                          const char* w_down, const char* b_down, const char* out, uint32_t in_dim,
                          uint32_t hidden_dim, uint32_t out_dim, vyb_program** program);
/* vyre-libs/src/nn/moe/moe_layer.rs:33 */
int32_t vyb_nn_moe_layer_route_and_accumulate(const char* x, const char* w_router, const char* b_router,
                                              const char* expert_indices, const char* expert_weights,
                                              const char* expert_outputs, const char* out, uint32_t in_dim,
                                              uint32_t num_experts, uint32_t out_dim, uint32_t k,
                                              vyb_program** program);

/* ---- serving-layout operators (no single reference builder; each composes the reference ops cited) --- */
/* Group-quantized int4 linear in the checkpoint-native layout: W packed u4 [out_dim, in_dim/2] K-inner
 * (the primitive word layout, programs.rs:181, read offset-binary with constant zero point 8), bf16 scale
 * [out_dim, in_dim/group], x bf16 [batch, in_dim], f32 accumulate, out bf16 or f32 [batch, out_dim].
 * Semantics = linear_4bit_affine_grouped (linear_4bit.rs:357) with zp == 8 and typed bf16 I/O
 * (linear_rows_no_bias_out_in_typed, builder.rs:241). Slots: x=0, w=1, scale=2, out=3. The backend picks the
 * decode GEMV for batch <= 8 and the tcgen05 prefill GEMM for large batches. op id
 * "vyre-b200::nn::linear_int4_grouped_rowmajor". */
int32_t vyb_nn_linear_int4_grouped_rowmajor(const char* x, const char* w_packed, const char* scale, const char* out,
                                            uint32_t batch, uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                            uint32_t out_dtype, vyb_program** program);
/* The same projection with its neighbours in the residual block taken into the node (dense_gated_mlp.rs:168-370: `mlp.norm`
 * in front of gate_proj / up_proj, `mlp.swiglu` behind up_proj, `mlp.residual` behind down_proj): a learned RMSNorm of x
 * (bf16 weight [in_dim], gated_rms_norm.rs:35-247 without gate) when `norm_weight` is named; behind the projection either
 * SwiGLU(gate, projection) (swiglu.rs:51-79; gate bf16 [batch, out_dim], the gate projection's output) when `gate` is
 * named, or a residual add (residual_add.rs:8-52; residual bf16 [batch, out_dim]) when `residual` is named - not both; at
 * least one part. bf16 throughout; every intermediate is rounded as the stand-alone operators round it, so the node's
 * values are those of the operators run in sequence. Slots in order: x, [norm_weight], w, scale, [gate | residual], out.
 * For one or two batch rows of 2048 / 4096 elements the decode GEMV does all of it in one launch (kernel variant 9); for
 * longer rows (up to four batch rows) SwiGLU / the residual add join the launch; other shapes run the stand-alone kernels
 * inside the node. No reference builder: the reference fuses neighbouring nodes in its megakernel scheduler. op id
 * "vyre-b200::nn::linear_int4_block". */
int32_t vyb_nn_linear_int4_block(const char* x, const char* norm_weight, const char* w_packed, const char* scale, const char* gate,
                                 const char* residual, const char* out, uint32_t batch, uint32_t in_dim, uint32_t out_dim,
                                 uint32_t group_size, float norm_eps, vyb_program** program);
/* int8 weight-only linear: W int8 [out_dim, in_dim], per-output-channel f32 scale, x/out f32;
 * = int8_unpack (int8.rs:15) with signed bytes + linear_rows_no_bias_out_in (builder.rs:241).
 * Slots: x=0, w=1, scale=2, out=3. op id "vyre-b200::nn::linear_int8_weight_only". */
int32_t vyb_nn_linear_int8_weight_only(const char* x, const char* w, const char* scale, const char* out,
                                       uint32_t batch, uint32_t in_dim, uint32_t out_dim, vyb_program** program);
/* Dynamic per-token int8 x int8 -> int32 linear: x bf16 [rows, in_dim] quantized per token
 * (s_t = max|x|/127, q = clamp(rne(x/s_t), -127, 127)), W int8 [out_dim, in_dim]; out int32 [rows, out_dim]
 * (= the wrapping-u32 Matmul, matmul.rs:17-60, on sign-extended bytes) and x_scale f32 [rows].
 * Slots: x=0, w=1, x_scale=2 (RW), out=3. op id "vyre-b200::nn::linear_int8_dynamic". */
int32_t vyb_nn_linear_int8_dynamic(const char* x, const char* w, const char* x_scale, const char* out, uint32_t rows,
                                   uint32_t in_dim, uint32_t out_dim, vyb_program** program);
/* Multi-token int4 MoE FFN layer: router linear (bf16 [experts, hidden]) -> moe_gate (gating.rs:19) per
 * token -> per selected expert swiglu_typed(w1 x, w3 x) (swiglu.rs:26) -> w2 -> weighted accumulate
 * (moe_layer.rs:33). Expert weights stacked: w13 u4 [E][2][inter][hidden/2], s13 bf16 [E][2][inter][hidden/g],
 * w2 u4 [E][hidden][inter/2], s2 bf16 [E][hidden][inter/g].
 * Slots: x=0, w_router=1, w13=2, s13=3, w2=4, s2=5, out=6 (bf16 [tokens, hidden]), routing_idx=7 (RW u32
 * [tokens, topk]), routing_w=8 (RW f32 [tokens, topk]). op id "vyre-b200::nn::moe_ffn_int4".
 * The device path needs hidden and inter multiples of 256, group a multiple of 64, experts <= 64, topk <= 8;
 * other shapes are UnsupportedFeature at materialisation. */
int32_t vyb_nn_moe_ffn_int4(const char* x, const char* w_router, const char* w13, const char* s13, const char* w2,
                            const char* s2, const char* out, const char* routing_idx, const char* routing_w,
                            uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t topk,
                            uint32_t group_size, vyb_program** program);

/* ---- Program accessors (vyre_foundation::ir::Program) ---------------------------------------------- */
const char* vyb_program_op_id(const vyb_program* p); /* outermost Region generator */
uint32_t vyb_program_buffer_count(const vyb_program* p);
int32_t vyb_program_buffer(const vyb_program* p, uint32_t index, vyb_buffer_decl* out);
void vyb_program_workgroup_size(const vyb_program* p, uint32_t out[3]);
/* 1 when the builder produced a trap program (vyre-primitives/src/lib.rs:83-98); such a program is
 * refused by vyb_compile with InvalidProgram. vyb_program_trap_message gives the builder's "Fix: ..." text. */
uint32_t vyb_program_is_trap(const vyb_program* p);
const char* vyb_program_trap_message(const vyb_program* p);
void vyb_program_fingerprint(const vyb_program* p, uint8_t out[32]); /* Program::fingerprint */
void vyb_program_free(vyb_program* p);

/* A program rebuilt from what a vyre Artifact carries: the op id (outermost Region generator) and the BufferDecls of
 * its Program. This is what the TargetCompiler facet calls, because TargetCompiler::compile(&Artifact)
 * (vyre-megakernel/src/target.rs:180-189, helper :253-322) is handed an Artifact, not builder arguments, and a
 * Program keeps its dimensions as IR literals. `op_spec` (nullable) is the op's dimensions in builder order, taken
 * from the Program's metadata map (docs/wire-format.md:104-111) when the producer attached them; without it the
 * dimensions are recovered from the buffer counts. Either way every declaration is cross-checked against the rebuilt
 * program (count, dtype, access per slot): a mismatch is InvalidProgram. Ops: linear_4bit, linear_4bit_affine_grouped
 * (spec in_dim, out_dim, group_size, batch), int4 [batched_]matvec_f32_scaled under both id families (spec batch, rows,
 * cols), moe_gate (spec num_experts, k), swiglu (spec n), int8_unpack (spec n, cols); others UnsupportedFeature. */
int32_t vyb_program_from_op(const char* op_id, const vyb_buffer_decl* decls, uint32_t n_decls, const uint32_t* op_spec,
                            uint32_t n_spec, vyb_program** program);

/* ---- compile: ProgramGraph::from_program + vyre_megakernel::compile (vyre-megakernel/src/lib.rs:832) -- */
int32_t vyb_compile(const vyb_program* program, vyb_artifact** artifact);
void vyb_artifact_digest(const vyb_artifact* a, uint8_t out[32]);
void vyb_artifact_free(vyb_artifact* a);

/* ---- TargetCompiler::compile (vyre-megakernel/src/target.rs:180-189; pure, needs no device) ----------- */
int32_t vyb_target_compile(const vyb_artifact* artifact, vyb_payload** payload);
void vyb_payload_digest(const vyb_payload* p, uint8_t out[32]);
void vyb_payload_neutral_artifact(const vyb_payload* p, uint8_t out[32]);
const char* vyb_payload_format(const vyb_payload* p);
/* Which hand-written kernel the payload's first launch module names: 0 = the kernel that replays the reference's
 * evaluation order, 1.. = the kernels chosen from the op spec at target-compile time (the CUDA payload of the reference
 * carries its PTX entry point in the same place: vyre-driver-cuda/src/backend/artifact_lifecycle.rs:69-130). */
uint32_t vyb_payload_kernel_variant(const vyb_payload* p);
/* TargetPayload::to_bytes / from_bytes (vyre-megakernel/src/envelope.rs); from_bytes re-authenticates */
int32_t vyb_payload_bytes(const vyb_payload* p, const uint8_t** bytes, size_t* len);
int32_t vyb_payload_from_bytes(const uint8_t* bytes, size_t len, vyb_payload** payload);
void vyb_payload_free(vyb_payload* p);

/* ---- ProgramGraph (vyre-foundation/src/ir_inner/model/program_graph.rs:20-648) -----------------------------------------
 * Executable Programs connected by typed values. Construction order is the topological schedule (add_node appends a
 * node after all of its producers). A ValueContract is dtype + shape + access + lifetime (:44-56; lifetimes in the
 * reference's order, :31-42); only statically known dimensions exist here (ShapeDim::Symbol is not rebuilt). Every port
 * is checked against the Program's buffer (:541-634: element type, element count, access) and against the value it
 * connects to (:343-360: dtype, shape, lifetime); names are unique over nodes and values; a buffer or a value is bound
 * once per node; a retained successor must consume and preserve the value it replaces (:363-384). Violations are
 * InvalidProgram errors that carry the reference's wording. vyb_graph_from_program is ProgramGraph::from_program
 * (:225-270); vyb_graph_value reports the value's liveness interval in schedule indices (:486-503). The graph is host
 * metadata: a runtime walks the schedule and submits one materialised Program per node, values bound as resident
 * buffers (the Python mirror's GraphSession does exactly that). */
#define VYB_LIFETIME_CONSTANT 0u
#define VYB_LIFETIME_INVOCATION 1u
#define VYB_LIFETIME_RETAINED 2u
#define VYB_LIFETIME_OUTPUT 3u
typedef struct vyb_graph vyb_graph;
typedef struct vyb_value_contract {
    uint32_t dtype;
    uint32_t access;   /* VYB_ACCESS_READ_ONLY or VYB_ACCESS_READ_WRITE (a declared output buffer is ReadWrite) */
    uint32_t lifetime; /* VYB_LIFETIME_* */
    uint32_t rank;
    uint64_t shape[6];
} vyb_value_contract;
typedef struct vyb_graph_input {
    const char* buffer; /* Program-local buffer name */
    uint32_t value;     /* connected graph value */
    vyb_value_contract contract;
} vyb_graph_input;
typedef struct vyb_graph_output {
    const char* buffer;
    const char* name; /* stable graph value name */
    vyb_value_contract contract;
    int64_t retained_successor_of; /* value id, or -1 */
} vyb_graph_output;
typedef struct vyb_graph_value_info {
    const char* name;
    vyb_value_contract contract;
    int64_t producer; /* node id, or -1 for external values */
    uint32_t n_consumers;
    int64_t retained_successor_of;
    uint32_t live_start, live_end;
} vyb_graph_value_info;
typedef struct vyb_graph_node_info {
    const char* name;
    const vyb_program* program; /* owned by the graph */
    uint32_t n_inputs, n_outputs;
} vyb_graph_node_info;
int32_t vyb_graph_new(vyb_graph** graph);
void vyb_graph_free(vyb_graph* g);
int32_t vyb_graph_add_external_value(vyb_graph* g, const char* name, const vyb_value_contract* contract, uint32_t* value_id);
int32_t vyb_graph_add_node(vyb_graph* g, const char* name, const vyb_program* program, const vyb_graph_input* inputs,
                           uint32_t n_inputs, const vyb_graph_output* outputs, uint32_t n_outputs, uint32_t* node_id,
                           uint32_t* output_value_ids);
int32_t vyb_graph_from_program(const char* node_name, const vyb_program* program, vyb_graph** graph);
uint32_t vyb_graph_node_count(const vyb_graph* g);
uint32_t vyb_graph_value_count(const vyb_graph* g);
int32_t vyb_graph_value(const vyb_graph* g, uint32_t id, vyb_graph_value_info* out);
int32_t vyb_graph_node(const vyb_graph* g, uint32_t id, vyb_graph_node_info* out);
int32_t vyb_graph_node_input(const vyb_graph* g, uint32_t node, uint32_t index, vyb_graph_input* out);
int32_t vyb_graph_node_output(const vyb_graph* g, uint32_t node, uint32_t index, vyb_graph_output* out, uint32_t* value_id);
void vyb_graph_digest(const vyb_graph* g, uint8_t out[32]);
/* A copy of the graph in which bf16 learned-RMSNorm nodes that feed only int4 row-major linears, a bf16 SwiGLU whose `up`
 * comes from such a linear, and a bf16 residual add whose `branch` does, are taken into vyb_nn_linear_int4_block nodes
 * wherever the decode kernel does the part in its own launch; all other nodes, names, contracts and the order are kept,
 * the values are unchanged. `n_fused` (nullable): how many nodes were taken in. The reference's counterpart is the fusion
 * step of its megakernel scheduler (vyre-megakernel: schedule search over fusion groups), which is not rebuilt; this pass
 * knows these three patterns only. */
int32_t vyb_graph_fuse_linear_blocks(const vyb_graph* g, vyb_graph** fused, uint32_t* n_fused);

/* ---- safetensors ingestion (vyre-safetensors/src/lib.rs:108-260, 871-907: SafetensorIndex::open) ---------------------
 * One shard's header, read and validated without touching tensor payloads: 8-byte prefix, header <= 64 MiB, a JSON
 * object of {dtype, shape, data_offsets} (`__metadata__` ignored, duplicate names refused), every range inside the
 * payload, byte length = shape x dtype width, no overlaps, at most 1 000 000 tensors, names of 1..4096 bytes. The
 * identity is (BLAKE3 of the exact header bytes, file length, payload start) as in SafetensorShardIdentity
 * (lib.rs:98-106). Entries come in canonical name order. dtype tags follow SafetensorDtype's declaration order
 * (BOOL 0, U8, I8, U16, I16, U32, I32, U64, I64, F16, BF16, F32, F64, F8_E4M3, F8_E5M2 14). vyb_safetensors_require is
 * SafetensorRequirement (lib.rs:262-271). vyb_safetensors_upload moves a tensor's bytes from the file into a resident
 * buffer (vyb_alloc) in bounded pieces through vyb_upload_at: weights then bind as resident values with the contract's
 * Constant lifetime. Sharded indexes and full-checkpoint content identities (lib.rs:330-640) are not rebuilt. */
typedef struct vyb_safetensors vyb_safetensors;
typedef struct vyb_safetensor_entry {
    const char* name;
    uint32_t dtype;
    const char* dtype_name;
    uint32_t rank;
    const uint64_t* shape;
    uint64_t file_begin, file_end; /* absolute byte range in the shard file */
} vyb_safetensor_entry;
int32_t vyb_safetensors_open(const char* path, vyb_safetensors** out);
void vyb_safetensors_free(vyb_safetensors* st);
void vyb_safetensors_identity(const vyb_safetensors* st, uint8_t header_digest[32], uint64_t* file_len, uint64_t* data_start);
uint32_t vyb_safetensors_count(const vyb_safetensors* st);
int32_t vyb_safetensors_entry(const vyb_safetensors* st, uint32_t index, vyb_safetensor_entry* out);
int32_t vyb_safetensors_find(const vyb_safetensors* st, const char* name, uint32_t* index);
int32_t vyb_safetensors_require(const vyb_safetensors* st, const char* name, const char* dtype_name, const uint64_t* shape,
                                uint32_t rank, uint32_t* index);

/* ---- Device (artifact_lifecycle.rs:21-30) + ArtifactMaterializer (artifact_lifecycle.rs:132-186) ------- */
int32_t vyb_device_acquire(int32_t ordinal, vyb_device** device);
int32_t vyb_device_identity_of(const vyb_device* d, vyb_device_identity* out);
int32_t vyb_device_caps_of(const vyb_device* d, vyb_device_caps* out);
int32_t vyb_device_is_healthy(const vyb_device* d);
/* Host-side loss injection for recovery tests: marks this generation lost exactly as a CUDA
 * context-loss error would (vyre-runtime/src/recovery.rs:13-25); no device fault is provoked. */
int32_t vyb_device_mark_lost(vyb_device* d, const char* reason);
/* Re-acquire after loss: returns a new generation on the same ordinal (ArtifactSession::rematerialize,
 * vyre-runtime/src/artifact_admission.rs:271-291, then re-admits the same payload bytes). */
int32_t vyb_device_reacquire(vyb_device* d);
void vyb_device_release(vyb_device* d);
/* a second owner of the same handle (the device stays acquired until every owner has released it) */
void vyb_device_retain(vyb_device* d);

/* resident buffers: vyre-driver-cuda/src/backend/resident.rs:138-201,426-443 */
int32_t vyb_alloc(vyb_device* d, size_t byte_len, vyb_resident_handle* out);
int32_t vyb_upload(vyb_device* d, vyb_resident_handle h, const void* bytes, size_t len);
int32_t vyb_upload_at(vyb_device* d, vyb_resident_handle h, size_t offset_bytes, const void* bytes, size_t len);
/* VyreBackend::download_resident / download_resident_range (vyre-driver/src/backend/vyre_backend.rs:298-381) */
int32_t vyb_download(vyb_device* d, vyb_resident_handle h, void* dst, size_t len);
int32_t vyb_download_range(vyb_device* d, vyb_resident_handle h, size_t offset_bytes, void* dst, size_t len);
int32_t vyb_free(vyb_device* d, vyb_resident_handle h);
/* a tensor of an indexed safetensors shard, file -> resident buffer at byte offset dst_offset */
int32_t vyb_safetensors_upload(const vyb_safetensors* st, uint32_t index, vyb_device* device, vyb_resident_handle handle,
                               uint64_t dst_offset);
/* raw device pointer of a resident buffer, for hosts that share the CUDA context */
int32_t vyb_resident_device_ptr(vyb_device* d, vyb_resident_handle h, void** device_ptr, size_t* len);

/* ArtifactMaterializer::materialize with the fail-closed checks of materialize::admit
 * (vyre-driver/src/materialize.rs:81-146) */
int32_t vyb_materialize(vyb_device* d, const vyb_artifact* artifact, const vyb_payload* payload,
                        vyb_instance** instance);
void vyb_instance_artifact_digest(const vyb_instance* i, uint8_t out[32]);
void vyb_instance_payload_digest(const vyb_instance* i, uint8_t out[32]);
int32_t vyb_instance_device(const vyb_instance* i, vyb_device_identity* out);
void vyb_instance_free(vyb_instance* i);

/* ArtifactInstance::submit (artifact_lifecycle.rs:120-129; CUDA impl vyre-driver-cuda/src/materializer.rs:165-283).
 * `artifact_digest` is BindingSet::artifact; a mismatch with the instance is InvalidProgram. Host and
 * resident bindings may be mixed (the reference's CUDA instance refuses that, materializer.rs:186-190; here
 * weights stay resident while activations arrive from the host). The launch is asynchronous on a
 * library-owned non-default stream. `config` may be NULL. */
int32_t vyb_submit(vyb_instance* instance, const uint8_t artifact_digest[32], const vyb_binding* bindings,
                   size_t n_bindings, const vyb_dispatch_config* config, vyb_submission** submission);
/* A binding set validated once and frozen into a single device-side graph (copy of the host inputs in, kernels,
 * copy of the outputs out; small outputs that a kernel writes completely are stored by the kernel straight into the
 * set's mapped pinned host buffer, and the status words live in a mapped pinned slot of the set), for a caller that submits the same artifact with the same
 * resident buffers over and over and only changes its host inputs. No counterpart in the reference, whose
 * ArtifactSession::submit (vyre-runtime/src/artifact_admission.rs:152-496) validates and stages every BindingSet
 * anew; the result of a replay equals that of vyb_submit with the same bindings. vyb_prepare runs one ordinary
 * submission first (full validation). vyb_prepared_submit copies the bytes of `host_updates` (host bindings of
 * input value ids; the others keep their last contents) and replays; one submission per prepared set may be in
 * flight: the completion's output views live in the set's buffers until the completion is freed. Resident
 * buffers bound to the set count as in flight (vyb_free refuses them) until vyb_prepared_free. */
int32_t vyb_prepare(vyb_instance* instance, const uint8_t artifact_digest[32], const vyb_binding* bindings,
                    size_t n_bindings, vyb_prepared** prepared);
int32_t vyb_prepared_submit(vyb_prepared* prepared, const vyb_binding* host_updates, size_t n_updates,
                            vyb_submission** submission);
/* The same, ordered on the device behind `after` (a pending submission of any instance of the same device; NULL: as
 * vyb_prepared_submit): the replay starts when `after` has completed, without the host waiting in between. A chain of
 * nodes (a ProgramGraph's schedule over resident values) is submitted back to back this way and waited for at the end;
 * the reference's CUDA Submission is synchronous (vyre-driver-cuda/src/materializer.rs:343-357) and has no such call.
 * Every submission still has to be waited for and its completion freed. */
int32_t vyb_prepared_submit_after(vyb_prepared* prepared, const vyb_submission* after, const vyb_binding* host_updates,
                                  size_t n_updates, vyb_submission** submission);
int32_t vyb_prepared_free(vyb_prepared* prepared);
/* Host-side injection for recovery tests, like vyb_device_mark_lost: writes `word` into the instance's kernel
 * status words exactly where a kernel whose bounded wait ran out would raise it; the NEXT submission on the
 * instance then fails with DispatchFailed and later ones succeed again. No device fault is provoked. */
int32_t vyb_instance_inject_status(vyb_instance* instance, uint32_t word);
/* Submission::is_ready / wait (artifact_lifecycle.rs:112-117); wait consumes the submission */
int32_t vyb_submission_is_ready(const vyb_submission* s);
int32_t vyb_submission_wait(vyb_submission* s, vyb_completion** completion);
/* Completion (artifact_lifecycle.rs:100-109): host bytes per output value, device_ns when measured */
int32_t vyb_completion_output(const vyb_completion* c, uint32_t value_id, const uint8_t** bytes, size_t* len);
uint32_t vyb_completion_output_count(const vyb_completion* c);
int32_t vyb_completion_device_ns(const vyb_completion* c, uint64_t* ns);
void vyb_completion_free(vyb_completion* c);

/* ---- the reference's authenticated wire frames -----------------------------------------------------------
 * vyre-megakernel frames its three layers alike (lib.rs:1326-1355, envelope.rs:763-860):
 *   magic[4] | schema u16 LE | body_len u32 LE | body (compact serde_json) | BLAKE3(domain | schema | body_len u64 | body)
 * layer 0: VMK0 neutral artifact (schema 4), 1: VTP0 target payload (schema 3), 2: VME0 envelope (schema 2).
 * vyb_frame_encode / _decode are the framing alone (decode runs the reference's checks in its order: length, magic,
 * schema, declared length, digest). vyb_payload_to_vtp0 writes this backend's payload as a TargetPayloadBody
 * (envelope.rs:182-192) bound to the neutral artifact digest the caller holds (Artifact::digest() of vyre's own
 * compiler); `value_ids` maps the program's bound buffers, in declaration order, to ArtifactValueIds (NULL: the
 * binding slots). vyb_envelope_to_vme0 wraps one neutral frame and payload frames as an EnvelopeBody
 * (envelope.rs:383-389) and refuses a payload bound to another artifact. The VMK0 body is the reference compiler's
 * output: it is authenticated and carried here, never produced. Frames handed out are freed with vyb_frame_free. */
int32_t vyb_frame_encode(uint32_t layer, const uint8_t* body, size_t body_len, uint8_t** frame, size_t* frame_len);
int32_t vyb_frame_decode(uint32_t layer, const uint8_t* frame, size_t frame_len, const uint8_t** body, size_t* body_len,
                         uint8_t digest[32]);
void vyb_frame_free(uint8_t* frame);
int32_t vyb_payload_to_vtp0(const vyb_payload* payload, const uint8_t neutral_artifact[32], uint32_t node_id,
                            const uint32_t* value_ids, uint32_t n_value_ids, uint8_t** frame, size_t* frame_len);
int32_t vyb_payload_from_vtp0(const uint8_t* frame, size_t frame_len, vyb_payload** payload, uint8_t neutral_artifact[32]);
int32_t vyb_envelope_to_vme0(const uint8_t* vmk0, size_t vmk0_len, const uint8_t* const* vtp0, const size_t* vtp0_len,
                             uint32_t n_payloads, uint8_t** frame, size_t* frame_len);
/* index 0: the neutral artifact's frame, 1..n: the payload frames; inner may be NULL to only authenticate and count */
int32_t vyb_envelope_from_vme0(const uint8_t* frame, size_t frame_len, uint32_t index, uint8_t** inner, size_t* inner_len,
                               uint32_t* n_payloads);

/* ---- scratch-reusing callers of the packed-int4 primitives -----------------------------------------------
 * vyre-self-substrate/src/math/quantized_dispatch.rs:30-90 and quantized_dispatch/{unpack,dot,matvec,batched_matvec,
 * batched_matmul,top1}.rs: the `*_via_with_scratch_into` functions. Host slices in (pointer + element count), host
 * slice out (the caller provides exactly the documented number of elements), the shape checks and `Fix:` texts of
 * the reference, one dispatch per call. The dispatcher is the device the scratch was made for. ONE scratch type
 * serves all six wrappers (the reference has one struct per wrapper, each a Program cache plus staging vectors): it
 * caches per (wrapper, shape) the Program, Artifact, TargetPayload and ArtifactInstance, so a repeated shape costs
 * one submission. Calls on one scratch are serialised. Errors: VYB_ERR_DISPATCH_*. A scratch made with a NULL device
 * validates shapes and refuses every dispatch (Rejected). */
typedef struct vyb_quantized_scratch vyb_quantized_scratch;
int32_t vyb_quantized_scratch_new(vyb_device* device, vyb_quantized_scratch** scratch);
void vyb_quantized_scratch_free(vyb_quantized_scratch* scratch);
void vyb_quantized_scratch_stats(const vyb_quantized_scratch* scratch, uint64_t* cached, uint64_t* hits, uint64_t* misses);
/* unpack.rs:36-84: out_lanes has lane_count i32 */
int32_t vyb_unpack_i4x8_via(vyb_quantized_scratch* scratch, const uint32_t* packed_words, size_t packed_len,
                            uint32_t lane_count, int32_t* out_lanes);
/* dot.rs:44-91: out has one f32 */
int32_t vyb_i4x8_dot_f32_scaled_via(vyb_quantized_scratch* scratch, const uint32_t* lhs_packed, size_t lhs_len,
                                    const uint32_t* rhs_packed, size_t rhs_len, float lhs_scale, float rhs_scale,
                                    uint32_t lane_count, float* out);
/* matvec.rs:45-110: out has rows f32 */
int32_t vyb_i4x8_matvec_f32_scaled_via(vyb_quantized_scratch* scratch, const uint32_t* weights_packed, size_t weights_len,
                                       const float* x, size_t x_len, const float* row_scales, size_t row_scales_len,
                                       uint32_t rows, uint32_t cols, float* out);
/* batched_matvec.rs:47-132: out has batch * rows f32 */
int32_t vyb_i4x8_batched_matvec_f32_scaled_via(vyb_quantized_scratch* scratch, const uint32_t* weights_packed,
                                               size_t weights_len, const float* x_batches, size_t x_len,
                                               const float* row_scales, size_t row_scales_len, uint32_t batch,
                                               uint32_t rows, uint32_t cols, float* out);
/* batched_matmul.rs:45-108 (shape rule shapes.rs:12-76): out has batch * rows f32 */
int32_t vyb_i4x8_batched_matmul_f32_scaled_via(vyb_quantized_scratch* scratch, const uint32_t* weights_packed,
                                               size_t weights_len, const uint32_t* activation_batches_packed,
                                               size_t activations_len, const float* row_scales, size_t row_scales_len,
                                               const float* batch_scales, size_t batch_scales_len, uint32_t batch,
                                               uint32_t rows, uint32_t cols, float* out);
/* top1.rs:44-126: scores_out and indices_out have batch elements each */
int32_t vyb_i4x8_batched_matmul_top1_f32_scaled_via(vyb_quantized_scratch* scratch, const uint32_t* weights_packed,
                                                    size_t weights_len, const uint32_t* activation_batches_packed,
                                                    size_t activations_len, const float* row_scales,
                                                    size_t row_scales_len, const float* batch_scales,
                                                    size_t batch_scales_len, uint32_t batch, uint32_t rows,
                                                    uint32_t cols, float* scores_out, uint32_t* indices_out);

/* ---- kernel-level entry points ------------------------------------------------------------------------
 * For a host that owns its buffers and stream (what the Rust shim's resident path calls after resolving
 * handles; replaces launch_cuda_function -> cuLaunchKernel, vyre-driver-cuda/src/backend/launch.rs:65-125).
 * All pointers are DEVICE pointers, `stream` is a cudaStream_t. `status` is an optional device pointer to
 * 4 u32 words that a kernel with bounded waits sets non-zero when a wait ran out (never a trap). */

/* Tensor-core peak microbenchmark (no counterpart in the reference: its bench reports no roofline for tensor
 * work, vyre-bench/src/api/metric.rs:109-118): every SM issues `iters` rounds of four tcgen05.mma (128 x 256 tiles,
 * kind::i8 when int8 != 0, else bf16) from operands resident in shared memory. *ops_per_launch receives the
 * integer or floating-point operations one launch performs; the caller times launches with events. */
int32_t vyb_k_tensor_peak(uint32_t int8, uint32_t iters, void* stream, uint32_t* status, double* ops_per_launch);
/* y[m,n] = bf16|f32( sum_k x[m,k] * (q[n,k]-8) * s[n,k/group] ), m <= 8 per pass, HBM-bound decode path.
 * group 128, k a multiple of 1024. Routing: k 2048 / 4096 with up to two rows (f32 outputs: one row per launch) runs
 * the half-SM integer kernel, three to eight rows one launch on the f16 tensor path; k a larger multiple of 2048 is
 * cut into k blocks inside one launch, which keeps a workspace per (device, stream) allocated on the first call that
 * is not under stream capture (a first call under capture runs one launch per k block with a stream-ordered scratch
 * allocation instead); other k run the bulk-copy kernel. Launches that share a stream are ordered; graphs captured
 * on one stream must not be replayed concurrently on two streams when they hold long-row launches (they share that
 * stream's workspace). */
int32_t vyb_k_int4_gemv(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                        uint32_t n, uint32_t k, uint32_t group_size, uint32_t out_dtype, void* stream,
                        uint32_t* status);
/* Same with launch flags. VYB_LAUNCH_CONSTANT_WEIGHTS: w_packed and scale_bf16 are constants of the graph
 * (ValueLifetime::Constant, vyre-libs/src/nn/model/dense_gated_mlp.rs:59-370), never written by a kernel that
 * precedes this launch in the stream; the kernel is then launched with programmatic stream serialization and
 * starts streaming them while the preceding kernel drains. Activations and outputs still wait for it. */
#define VYB_LAUNCH_CONSTANT_WEIGHTS 1u
/* Launch on one SM fewer than the device has, so that a small kernel of another stream (vyb_k_allgather_push) finds
 * an SM whose memory pipeline is not saturated by the weight stream. */
#define VYB_LAUNCH_LEAVE_ONE_SM 2u
int32_t vyb_k_int4_gemv_ex(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                           uint32_t n, uint32_t k, uint32_t group_size, uint32_t out_dtype, uint32_t flags,
                           void* stream, uint32_t* status);
/* The decode projection with its neighbours of the residual block in the same launch (the kernel behind
 * vyb_nn_linear_int4_block, kernel variant 9): y = f(W a) with a = rmsnorm(x) * norm_weight or a = x, and f = SwiGLU(gate, .)
 * or f = residual + . or the identity; bf16 throughout, rounded where the stand-alone operators round. norm_weight_bf16
 * [k], gate_bf16 [m, n] and residual_bf16 [m, n] are nullable (at least one given, not gate and residual together).
 * Shapes: group 128 and either m <= 2 with k 2048 / 4096 (every part), or no norm with m <= 4 and k a larger multiple of
 * 2048 (SwiGLU / the residual where the last k block rounds the sums; on a stream that captures before its first plain use
 * of the shape, a kernel of its own follows instead). flags as for vyb_k_int4_gemv_ex. Other shapes: UnsupportedFeature. */
int32_t vyb_k_int4_linear_block(const void* x_bf16, const void* norm_weight_bf16, float norm_eps, const void* w_packed,
                                const void* scale_bf16, const void* gate_bf16, const void* residual_bf16, void* y_bf16, uint32_t m,
                                uint32_t n, uint32_t k, uint32_t group_size, uint32_t flags, void* stream, uint32_t* status);
/* The stand-alone neighbours on raw device pointers (the kernels behind vyb_nn_learned_rms_norm, vyb_nn_residual_add_typed
 * and vyb_nn_swiglu_typed); dtype F16, BF16 or F32. The norm uses the long-row form from 2048 elements on. */
int32_t vyb_k_rms_norm(const void* input, const void* weight, void* output, uint32_t rows, uint32_t hidden, float eps,
                       uint32_t dtype, void* stream);
int32_t vyb_k_residual_add(const void* residual, const void* branch, void* output, uint32_t n, uint32_t dtype, void* stream);
int32_t vyb_k_swiglu(const void* gate, const void* up, void* output, uint32_t n, uint32_t dtype, void* stream);
/* All-gather of column-parallel outputs over peer memory (NVLink), one process per GPU (no counterpart in the
 * reference, whose backends are single-device; the sharding follows from its one-output-per-invocation kernels,
 * vyre-libs/src/nn/linear/inner/linear_4bit.rs:710-742). Every rank owns a gather buffer [2][world][m][n] bf16 that
 * all ranks can address. A plain GEMV (vyb_k_int4_gemv_ex) writes this rank's [m, n] slice into half `half` of the
 * local buffer (peer_out[rank] + ((half * world + rank) * m * n) elements); vyb_k_allgather_push copies it to every
 * peer, bumps their arrival counters and advances the local launch counter. Halves alternate; before a push
 * overwrites a half it checks (bounded) that every peer has completed all earlier pushes, so a consumer of the
 * gathered [world][m][n] must run, on every rank, before that rank's next push, after vyb_k_allgather_wait - which
 * waits (bounded, ~2 s, status bit 128) until every gather pushed so far by this rank is complete in local memory.
 * On a side stream the push overlaps the next GEMV; the caller orders it after the GEMV that wrote the slice and
 * before the GEMV that overwrites that half again. The buffer may hold more than two such slots ([slots][world][m][n],
 * `half` then is the slot index): a chain of GEMVs that each write a slot of their own needs no edge back from the
 * pushes into the chain, so consecutive GEMVs keep their programmatic dependency (the push CTAs, 128 threads at no
 * more than 32 registers, become resident beside the GEMV's).
 * peer_out / peer_flag: device addresses valid on THIS rank for every rank's buffer / 256 bytes of arrival counters
 * (own rank included); epoch: eight local 32-bit words. All counters zero before the first push. m * n a multiple of
 * 8. One CTA per peer copies, fences and signals, so a push costs the same at 2 and at 8 ranks. */
typedef struct vyb_allgather_ctx {
    uint32_t world, rank;
    uint64_t peer_out[8];
    uint64_t peer_flag[8];   /* 256 bytes of counters per rank: 32-bit word 8*s counts the pushes received from rank s */
    uint64_t epoch;          /* 16 local 32-bit words, zero before the first launch */
    uint64_t wait_clocks;    /* clock limit of a device-side wait (status bit 128 when it runs out); 0 = about 2 s */
    uint64_t slots;          /* slots of the gather buffer; 0 = the two halves. A push into slot s waits only until every peer
                              * has completed all but the last slots - 2 of the pushes this rank has completed */
} vyb_allgather_ctx;
int32_t vyb_k_allgather_push(const vyb_allgather_ctx* ctx, uint32_t half, uint32_t m, uint32_t n, void* stream,
                             uint32_t* status);
int32_t vyb_k_allgather_wait(const vyb_allgather_ctx* ctx, void* stream, uint32_t* status);
/* The decode GEMV of a column-parallel shard and its all-gather in ONE launch (no counterpart in the reference): the
 * reduction that produces an output stores it, as bf16, into this rank's [m, n] slice of buffer half `half` on every
 * rank (peer stores over NVLink; same buffers and counters as vyb_k_allgather_push). Consecutive launches stay one
 * programmatic chain (VYB_LAUNCH_CONSTANT_WEIGHTS), nothing runs on a side stream, and no CTA fences at system scope:
 * the arrival signal of a launch is sent by the next launch of this kind or by vyb_k_allgather_wait, which a stream
 * must run before it reads a gathered result. Halves must alternate from launch to launch; before it overwrites a
 * half on a peer a launch checks (bounded, status bit 128) that the peer has signalled its previous launch. epoch must
 * point to 16 zeroed local words. 1 <= m <= 4, group 128, k 2048 or 4096.
 * VYB_LAUNCH_PIPELINED_GATHER: a launch cannot end before its peer stores have drained (an NVLink round trip), which
 * delays the next launch of a dependent chain. With this flag a launch stores its outputs into the LOCAL buffer only;
 * the NEXT launch of this kind (same m and n) carries them to the peers right after its dependency wait, so that the
 * stores drain under its own work, and vyb_k_allgather_wait carries the last slice over. A gathered result is complete
 * one launch later. Do not mix flagged and unflagged launches between two waits. */
int32_t vyb_k_int4_gemv_allgather(const vyb_allgather_ctx* ctx, uint32_t half, const void* x_bf16, const void* w_packed,
                                  const void* scale_bf16, uint32_t m, uint32_t n, uint32_t k, uint32_t group_size,
                                  uint32_t flags, void* stream, uint32_t* status);
/* Column-parallel gather of a block of rows over peer memory (no counterpart in the reference; same sharding
 * argument as above). peer_out[r] is the base of rank r's full [M, N] output; this rank's block [rows, row_bytes]
 * (its columns of some rows, e.g. the int32 outputs of one M-chunk of its GEMM shard) is stored at byte offset
 * dst_offset_bytes (row pitch dst_pitch_bytes) of EVERY rank's output, own rank included, 16 CTAs per
 * destination side by side; then every destination's counter for this rank goes up by one. Chunks over M let the
 * gather of one chunk (on a side stream) overlap the GEMM of the next. epoch must point to 16 zeroed local words.
 * vyb_k_colpar_wait: bounded device-side wait until every rank has delivered `blocks` blocks into this rank's
 * output. Offsets, pitch and row bytes are multiples of 16. */
int32_t vyb_k_colpar_push(const vyb_allgather_ctx* ctx, const void* block, uint32_t rows, uint32_t row_bytes,
                          uint64_t dst_pitch_bytes, uint64_t dst_offset_bytes, void* stream, uint32_t* status);
int32_t vyb_k_colpar_wait(const vyb_allgather_ctx* ctx, uint32_t blocks, void* stream, uint32_t* status);
/* The int8 GEMM of a column-parallel shard and the gather of its int32 outputs in ONE kernel (no counterpart in the
 * reference): the epilogue that reads a tile's accumulators out of tensor memory stores them at byte offset
 * dst_offset_bytes (row pitch dst_pitch_bytes) of EVERY rank's full output peer_out[r] - plain 16-byte peer stores over
 * NVLink for the other ranks - while the MMA warp is already on the next tile, so the transfer overlaps the math tile
 * by tile and no copy kernel or staging buffer exists. A one-warp kernel behind it in the stream raises every
 * destination's counter for this rank by one (one block delivered); vyb_k_colpar_wait is the consumer-side check as
 * before. m > 128 (the paired tcgen05 kernel), n a multiple of 4. */
int32_t vyb_k_int8_gemm_i32_gather(const vyb_allgather_ctx* ctx, const void* a_i8, const void* w_i8, uint32_t m, uint32_t n,
                                   uint32_t k, uint64_t dst_pitch_bytes, uint64_t dst_offset_bytes, void* stream,
                                   uint32_t* status);

/* C1: y f32 [m,n] = x f32 [m,k] . (int8 w[n,k] * s[n])^T */
int32_t vyb_k_int8_weight_only_linear(const void* x_f32, const void* w_i8, const void* scale_f32, void* y_f32,
                                      uint32_t m, uint32_t n, uint32_t k, void* stream);

/* Prefill GEMM: y[m,n] = bf16|f32( sum_k x[m,k] * bf16((q[n,k]-8) * s[n,k/group]) ), weights dequantised to bf16
 * tiles inside the kernel and contracted on tcgen05 (f32 accumulate in TMEM). Same operands and layout as
 * vyb_k_int4_gemv, any m; k and group multiples of 64. */
int32_t vyb_k_int4_prefill_gemm(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                uint32_t n, uint32_t k, uint32_t group_size, uint32_t out_dtype, void* stream,
                                uint32_t* status);
/* Per-token symmetric int8 quantisation of bf16 rows: s_t = max|x_t| / 127, q = clamp(rint(x / s_t), -127, 127).
 * No reference builder quantises activations; the rule is this backend's (see vyb_nn_linear_int8_dynamic). */
int32_t vyb_k_quantize_per_token_int8(const void* x_bf16, void* q_i8, void* scales_f32, uint32_t m, uint32_t k,
                                      void* stream);
/* out int32 [m,n] = a int8 [m,k] . w int8 [n,k]^T on tcgen05 (kind::i8, s32 accumulate in TMEM); the signed
 * reading of the reference's wrapping-u32 Matmul (vyre-libs/src/math/linalg/matmul.rs:17-60). k % 16 == 0. */
int32_t vyb_k_int8_gemm_i32(const void* a_i8, const void* w_i8, void* out_i32, uint32_t m, uint32_t n, uint32_t k,
                            void* stream, uint32_t* status);
/* Same with launch flags. VYB_LAUNCH_LEAVE_COPY_SMS: the persistent GEMM runs on 16 SMs fewer than the device has, so
 * that a copy kernel of another stream (vyb_k_colpar_push of the previous row chunk) runs beside it instead of
 * behind it. */
#define VYB_LAUNCH_LEAVE_COPY_SMS 4u
#define VYB_LAUNCH_PIPELINED_GATHER 8u /* vyb_k_int4_gemv_allgather: see there */
int32_t vyb_k_int8_gemm_i32_ex(const void* a_i8, const void* w_i8, void* out_i32, uint32_t m, uint32_t n, uint32_t k,
                               uint32_t flags, void* stream, uint32_t* status);
/* The fused multi-token MoE FFN layer of vyb_nn_moe_ffn_int4 on raw device pointers (same operands, layouts and
 * results; batched composition of vyre-libs/src/nn/moe/{gating.rs:19,expert_mlp.rs:18,moe_layer.rs:33}). The caller
 * provides the scratch (expert-sorted rows, hidden activations, per-pair outputs, routing plan); its size comes
 * from vyb_k_moe_ffn_int4_scratch_bytes. routing_idx u32 [tokens, topk] and routing_w f32 [tokens, topk] are
 * outputs. hidden and inter multiples of 256, group a multiple of 64, experts <= 64, topk <= 8. */
int32_t vyb_k_moe_ffn_int4_scratch_bytes(uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts,
                                         uint32_t topk, uint64_t* bytes);
int32_t vyb_k_moe_ffn_int4(const void* x_bf16, const void* w_router_bf16, const void* w13, const void* s13, const void* w2,
                           const void* s2, void* out_bf16, void* routing_idx, void* routing_w, void* scratch,
                           uint64_t scratch_bytes, uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts,
                           uint32_t topk, uint32_t group_size, void* stream, uint32_t* status);
/* The stages of that layer on their own, for expert-parallel runs that exchange rows between them (all-to-all):
 *   vyb_k_moe_route         router linear + moe_gate per token (gating.rs:19): routing_idx u32 / routing_w f32 [tokens, topk]
 *   vyb_k_rows_gather_bf16  dst[i,:] = src[index[i],:] for bf16 rows (row_elems % 8 == 0); index 0xFFFFFFFF gives a zero row
 *   vyb_k_moe_experts_int4  swiglu(W1 x, W3 x) then W2 (expert_mlp.rs:18) for expert-sorted rows whose per-expert
 *                           segments are padded to 256 rows: tile_expert[i] = expert of rows [256 i, 256 i + 256),
 *                           *m_tiles = number of such tiles (both in device memory), h_scratch bf16 [max_rows, inter]
 *   vyb_k_moe_combine       out[t,:] = bf16(sum_j routing_w[t,j] * y_rows[pos[t,j],:]) (moe_layer.rs:33) */
int32_t vyb_k_moe_route(const void* x_bf16, const void* w_router_bf16, void* routing_idx, void* routing_w, uint32_t tokens,
                        uint32_t hidden, uint32_t experts, uint32_t topk, void* stream);
int32_t vyb_k_rows_gather_bf16(const void* src, const void* index_u32, void* dst, uint32_t rows, uint32_t row_elems,
                               void* stream);
int32_t vyb_k_moe_experts_int4(const void* x_sorted, const void* w13, const void* s13, const void* w2, const void* s2,
                               void* y_rows, void* h_scratch, const void* tile_expert_u32, const void* m_tiles_u32,
                               uint32_t max_rows, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t group_size,
                               void* stream, uint32_t* status);
int32_t vyb_k_moe_combine(const void* y_rows, const void* pos_u32, const void* routing_w, void* out_bf16, uint32_t tokens,
                          uint32_t hidden, uint32_t topk, void* stream);
/* Expert-parallel form of the MoE FFN layer, one process per GPU, with dispatch and combine done by this library's
 * kernels over peer memory (NVLink) - no host read-back, no NCCL call inside the layer (no counterpart in the
 * reference, whose backends are single-device; experts are independent programs, expert_mlp.rs:18-150, routing is
 * per token, gating.rs:19-69). Rank r owns experts [r * E / world, (r + 1) * E / world): w13 / s13 / w2 / s2 hold only
 * those. Every rank passes its own tokens; results and routing come back for exactly those tokens. The call is
 * collective: every rank must enqueue it the same number of times. Device-side waits are bounded (~2 s, status bit
 * 256). vyb_k_moe_ep_sizes fills the offsets of ctx and returns the byte sizes of the symmetric region (allocated
 * so that every rank can address every peer's copy, zero-filled; peer_base[r] = its address as seen from this rank)
 * and of the local scratch (zero-filled once); tokens_total bounds the rows that can land on one rank. */
typedef struct vyb_moe_ep_ctx {
    uint32_t world, rank;
    uint64_t peer_base[8];
    uint64_t off_counts, off_flags, off_src, off_xg, off_yhome;
    uint64_t wait_clocks; /* clock limit of a device-side wait (status bit 256 when it runs out); 0 = about 2 s */
} vyb_moe_ep_ctx;
int32_t vyb_k_moe_ep_sizes(uint32_t tokens_local_max, uint32_t tokens_total, uint32_t hidden, uint32_t inter,
                           uint32_t experts, uint32_t topk, uint32_t world, vyb_moe_ep_ctx* ctx, uint64_t* symmetric_bytes,
                           uint64_t* local_bytes);
int32_t vyb_k_moe_ep_ffn_int4(const vyb_moe_ep_ctx* ctx, const void* x_bf16, const void* w_router_bf16, const void* w13,
                              const void* s13, const void* w2, const void* s2, void* out_bf16, void* routing_idx,
                              void* routing_w, void* local_scratch, uint32_t tokens, uint32_t tokens_total, uint32_t hidden,
                              uint32_t inter, uint32_t experts, uint32_t topk, uint32_t group_size, void* stream,
                              uint32_t* status);
/* No counterpart in the reference. vyb_k_quantize_per_token_int8 followed by vyb_k_int8_gemm_i32 (x_scale_f32 [m],
 * y_i32 [m,n]) for callers that must not allocate device memory: the quantised activations go to a fixed 8 MiB
 * device array that belongs to the loaded library, so m * k <= 8388608 (larger shapes are InvalidProgram). All
 * calls on a device share that array: overlapping calls (two streams, two threads) race, so serialise them on
 * one stream. The first call on each device looks the array's address up; make it during set-up, before any
 * stream capture. */
int32_t vyb_k_linear_int8_dynamic_static_scratch(const void* x_bf16, const void* w_i8, void* x_scale_f32, void* y_i32,
                                                 uint32_t m, uint32_t n, uint32_t k, void* stream, uint32_t* status);
#define VYB_STATIC_SCRATCH_BYTES 8388608u

#ifdef __cplusplus
}
#endif
#endif /* VYRE_B200_H */
