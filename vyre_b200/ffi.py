"""ctypes binding of libvyre_b200.so (the C ABI declared in include/vyre_b200.h).

The library is the product; this module only loads it and gives every export its signature. Loading fails
loudly when the library has not been built: there is no Python or CPU fallback for any operator.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libvyre_b200.so")

# DataType tags (vyre-spec/src/data_type.rs:227-257)
DT_U32, DT_I32, DT_F16, DT_BF16, DT_F32, DT_U8, DT_I8, DT_I4 = 0x01, 0x02, 0x09, 0x0A, 0x0B, 0x0E, 0x10, 0x1B
ACCESS_READ_ONLY, ACCESS_READ_WRITE, ACCESS_OUTPUT, ACCESS_WORKGROUP = 0, 1, 2, 3
BIND_HOST, BIND_RESIDENT = 0, 1
LAUNCH_CONSTANT_WEIGHTS = 1
LAUNCH_LEAVE_ONE_SM = 2
LAUNCH_LEAVE_COPY_SMS = 4
LAUNCH_PIPELINED_GATHER = 8

ERR_DEVICE_OUT_OF_MEMORY = 1001
ERR_UNSUPPORTED_FEATURE = 1002
ERR_DISPATCH_FAILED = 1005
ERR_INVALID_PROGRAM = 1006
ERR_DEVICE_LOST = 1008
ERR_DISPATCH_REJECTED, ERR_DISPATCH_BAD_INPUTS, ERR_DISPATCH_BACKEND = 2001, 2002, 2003


class BackendError(RuntimeError):
    """vyre_driver::BackendError: `code` is ErrorCode::stable_id, the message always carries 'Fix:'."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


class AllGatherCtx(C.Structure):
    """vyb_allgather_ctx: peer addresses of the gather buffers / arrival counters and the local step words."""

    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("peer_out", C.c_uint64 * 8), ("peer_flag", C.c_uint64 * 8),
                ("epoch", C.c_uint64), ("wait_clocks", C.c_uint64), ("slots", C.c_uint64)]


class MoeEpCtx(C.Structure):
    """vyb_moe_ep_ctx: peer addresses of the symmetric regions and the offsets inside them."""

    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("peer_base", C.c_uint64 * 8), ("off_counts", C.c_uint64),
                ("off_flags", C.c_uint64), ("off_src", C.c_uint64), ("off_xg", C.c_uint64), ("off_yhome", C.c_uint64),
                ("wait_clocks", C.c_uint64)]


class ResidentHandle(C.Structure):
    _fields_ = [("owner", C.c_uint64), ("id", C.c_uint64)]


class TargetProfile(C.Structure):
    _fields_ = [("identity", C.c_char * 64), ("generation", C.c_uint32), ("max_workgroup_size", C.c_uint32 * 3),
                ("max_invocations", C.c_uint32), ("max_dynamic_shared_bytes", C.c_uint32),
                ("subgroup_size", C.c_uint32)]


class RegistrationInfo(C.Structure):
    _fields_ = [("id", C.c_char_p), ("target_id", C.c_char_p), ("payload_format", C.c_char_p),
                ("format_version", C.c_uint32), ("precedence", C.c_uint32), ("profile", TargetProfile)]


class DeviceIdentity(C.Structure):
    _fields_ = [("backend", C.c_char * 32), ("device", C.c_char * 96), ("generation", C.c_uint64)]


class DeviceCaps(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("ordinal", C.c_int32), ("compute_major", C.c_int32),
                ("compute_minor", C.c_int32), ("total_memory", C.c_uint64), ("max_threads_per_block", C.c_int32),
                ("shared_memory_per_block", C.c_int32), ("shared_memory_per_sm", C.c_int32),
                ("shared_memory_per_block_optin", C.c_int32), ("warp_size", C.c_int32),
                ("cooperative_launch", C.c_int32), ("multi_processor_count", C.c_int32), ("l2_cache_bytes", C.c_int32),
                ("memory_clock_rate_khz", C.c_int32), ("core_clock_rate_khz", C.c_int32),
                ("global_memory_bus_width_bits", C.c_int32)]


class BufferDecl(C.Structure):
    _fields_ = [("name", C.c_char_p), ("binding", C.c_uint32), ("access", C.c_uint32), ("dtype", C.c_uint32),
                ("count", C.c_uint32), ("has_output_byte_range", C.c_uint32), ("output_byte_begin", C.c_uint64),
                ("output_byte_end", C.c_uint64)]


class QuantizedLinear4BitSpec(C.Structure):
    _fields_ = [("in_dim", C.c_uint32), ("out_dim", C.c_uint32), ("storage_dtype", C.c_uint32),
                ("scale_group_size", C.c_uint32), ("zero_point_group_size", C.c_uint32)]


class PlannerEvidence(C.Structure):
    _fields_ = [("in_dim", C.c_uint32), ("out_dim", C.c_uint32), ("group_size", C.c_uint32),
                ("group_count", C.c_uint32), ("packed_weight_bytes", C.c_uint64),
                ("dequantized_weight_bytes", C.c_uint64), ("sidecar_bytes", C.c_uint64), ("bias_bytes", C.c_uint64),
                ("output_bytes", C.c_uint64), ("dequant_bytes_elided", C.c_uint64), ("matmul_m", C.c_uint32),
                ("matmul_k", C.c_uint32), ("matmul_n", C.c_uint32), ("matmul_tile", C.c_uint32),
                ("matmul_selected_path", C.c_char_p), ("matmul_candidate_path", C.c_char_p),
                ("matmul_fallback_reason", C.c_char_p), ("tensor_core_eligible", C.c_uint32),
                ("output_drift_abs_tolerance", C.c_float)]


class ValueContract(C.Structure):
    _fields_ = [("dtype", C.c_uint32), ("access", C.c_uint32), ("lifetime", C.c_uint32), ("rank", C.c_uint32), ("shape", C.c_uint64 * 6)]


class GraphInput(C.Structure):
    _fields_ = [("buffer", C.c_char_p), ("value", C.c_uint32), ("contract", ValueContract)]


class GraphOutput(C.Structure):
    _fields_ = [("buffer", C.c_char_p), ("name", C.c_char_p), ("contract", ValueContract), ("retained_successor_of", C.c_int64)]


class GraphValueInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("contract", ValueContract), ("producer", C.c_int64), ("n_consumers", C.c_uint32),
                ("retained_successor_of", C.c_int64), ("live_start", C.c_uint32), ("live_end", C.c_uint32)]


class GraphNodeInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("program", C.c_void_p), ("n_inputs", C.c_uint32), ("n_outputs", C.c_uint32)]


LIFETIME_CONSTANT, LIFETIME_INVOCATION, LIFETIME_RETAINED, LIFETIME_OUTPUT = 0, 1, 2, 3


class SafetensorEntry(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_uint32), ("dtype_name", C.c_char_p), ("rank", C.c_uint32),
                ("shape", C.POINTER(C.c_uint64)), ("file_begin", C.c_uint64), ("file_end", C.c_uint64)]


class Binding(C.Structure):
    _fields_ = [("value_id", C.c_uint32), ("kind", C.c_int32), ("host_ptr", C.c_void_p), ("len", C.c_size_t),
                ("resident", ResidentHandle)]


class DispatchConfig(C.Structure):
    _fields_ = [("grid_override", C.c_uint32 * 3), ("workgroup_override", C.c_uint32 * 3), ("timeout_ns", C.c_uint64),
                ("label", C.c_char_p), ("ulp_budget", C.c_uint32), ("max_output_bytes", C.c_uint64),
                ("cooperative", C.c_uint32), ("leave_resident", C.c_uint32)]


_lib = None
_S, _U, _P, _PP = C.c_char_p, C.c_uint32, C.c_void_p, C.POINTER(C.c_void_p)

# name -> argtypes for every status-returning export (restype int32)
_STATUS_FUNCS = {
    "vyb_registration": [C.POINTER(RegistrationInfo)],
    "vyb_nn_linear_4bit": [_S, _S, _S, _S, _U, _U, _PP],
    "vyb_nn_linear_4bit_affine_grouped": [_S] * 6 + [_U] * 3 + [_PP],
    "vyb_nn_linear_4bit_affine_grouped_batched": [_S] * 6 + [_U] * 4 + [_PP],
    "vyb_nn_linear_4bit_affine_grouped_typed": [C.POINTER(QuantizedLinear4BitSpec)] + [_S] * 6 + [_PP],
    "vyb_nn_linear_4bit_affine_grouped_batched_typed": [C.POINTER(QuantizedLinear4BitSpec), _U] + [_S] * 6 + [_PP],
    "vyb_nn_linear_4bit_affine_grouped_planner_evidence": [C.POINTER(QuantizedLinear4BitSpec),
                                                            C.POINTER(PlannerEvidence)],
    "vyb_math_unpack_i4x8": [_S, _S, _U, _PP],
    "vyb_math_i4x8_dot_i32": [_S, _S, _S, _U, _U, _PP],
    "vyb_math_i4x8_dot_f32_scaled": [_S] * 5 + [_U, _U, _PP],
    "vyb_math_i4x8_matvec_f32_scaled": [_S] * 4 + [_U, _U, _U, _PP],
    "vyb_math_i4x8_batched_matvec_f32_scaled": [_S] * 4 + [_U] * 4 + [_PP],
    "vyb_math_i4x8_batched_matmul_f32_scaled": [_S] * 5 + [_U] * 4 + [_PP],
    "vyb_math_i4x8_batched_matmul_top1_f32_scaled": [_S] * 5 + [_U] * 4 + [_PP],
    "vyb_quant_int8_unpack": [_S, _S, _S, _U, _U, _PP],
    "vyb_quant_int8_pack": [_S, _S, _U, _PP],
    "vyb_nn_linear_rows": [_S] * 4 + [_U] * 3 + [_PP],
    "vyb_nn_linear_rows_no_bias": [_S] * 3 + [_U] * 3 + [_PP],
    "vyb_nn_linear_rows_no_bias_typed": [_S] * 3 + [_U] * 4 + [_PP],
    "vyb_nn_linear_rows_no_bias_out_in_typed": [_S] * 3 + [_U] * 4 + [_PP],
    "vyb_math_matmul": [_S] * 3 + [_U] * 3 + [_PP],
    "vyb_math_matmul_bias": [_S] * 4 + [_U] * 3 + [_PP],
    "vyb_math_matmul_bias_tiled": [_S] * 4 + [_U] * 4 + [_PP],
    "vyb_nn_linear": [_S] * 4 + [_U] * 2 + [_PP],
    "vyb_nn_linear_tiled": [_S] * 4 + [_U] * 3 + [_PP],
    "vyb_nn_moe_gate": [_S] * 3 + [_U, _U, _PP],
    "vyb_nn_softmax_top_k": [_S] * 3 + [_U, _U, _PP],
    "vyb_nn_top_k": [_S, _S, _U, _U, _PP],
    "vyb_nn_swiglu": [_S] * 3 + [_U, _PP],
    "vyb_nn_swiglu_typed": [_S] * 3 + [_U, _U, _PP],
    "vyb_nn_residual_add": [_S] * 3 + [_U, _PP],
    "vyb_nn_residual_add_typed": [_S] * 3 + [_U, _U, _PP],
    "vyb_nn_learned_rms_norm": [_S] * 3 + [_U, _U, C.c_float, _U, _PP],
    "vyb_nn_gated_rms_norm": [_S] * 4 + [_U, _U, C.c_float, _U, _PP],
    "vyb_nn_gated_rms_norm_with_weight_dtype": [_S] * 4 + [_U, _U, C.c_float, _U, _U, _PP],
    "vyb_quant_q4_k_unpack": [_S] * 4 + [_U, _PP],
    "vyb_quant_q2_k_unpack": [_S] * 4 + [_U, _PP],
    "vyb_quant_q4_k_linear": [_S] * 6 + [_U, _U, _PP],
    "vyb_quant_q2_k_linear": [_S] * 6 + [_U, _U, _PP],
    "vyb_nn_expert_mlp": [_S] * 8 + [_U] * 3 + [_PP],
    "vyb_nn_moe_layer_route_and_accumulate": [_S] * 7 + [_U] * 4 + [_PP],
    "vyb_nn_linear_int4_grouped_rowmajor": [_S] * 4 + [_U] * 5 + [_PP],
    "vyb_nn_linear_int4_block": [_S] * 7 + [_U] * 4 + [C.c_float, _PP],
    "vyb_nn_linear_int8_weight_only": [_S] * 4 + [_U] * 3 + [_PP],
    "vyb_nn_linear_int8_dynamic": [_S] * 4 + [_U] * 3 + [_PP],
    "vyb_nn_moe_ffn_int4": [_S] * 9 + [_U] * 6 + [_PP],
    "vyb_program_buffer": [_P, _U, C.POINTER(BufferDecl)],
    "vyb_program_from_op": [_S, C.POINTER(BufferDecl), _U, C.POINTER(C.c_uint32), _U, _PP],
    "vyb_graph_new": [_PP],
    "vyb_graph_add_external_value": [_P, _S, C.POINTER(ValueContract), C.POINTER(C.c_uint32)],
    "vyb_graph_add_node": [_P, _S, _P, C.POINTER(GraphInput), _U, C.POINTER(GraphOutput), _U, C.POINTER(C.c_uint32),
                           C.POINTER(C.c_uint32)],
    "vyb_graph_from_program": [_S, _P, _PP],
    "vyb_graph_fuse_linear_blocks": [_P, _PP, C.POINTER(C.c_uint32)],
    "vyb_graph_value": [_P, _U, C.POINTER(GraphValueInfo)],
    "vyb_graph_node": [_P, _U, C.POINTER(GraphNodeInfo)],
    "vyb_graph_node_input": [_P, _U, _U, C.POINTER(GraphInput)],
    "vyb_graph_node_output": [_P, _U, _U, C.POINTER(GraphOutput), C.POINTER(C.c_uint32)],
    "vyb_safetensors_open": [_S, _PP],
    "vyb_safetensors_entry": [_P, _U, C.POINTER(SafetensorEntry)],
    "vyb_safetensors_find": [_P, _S, C.POINTER(C.c_uint32)],
    "vyb_safetensors_require": [_P, _S, _S, C.POINTER(C.c_uint64), _U, C.POINTER(C.c_uint32)],
    "vyb_safetensors_upload": [_P, _U, _P, ResidentHandle, C.c_uint64],
    "vyb_quantized_scratch_new": [_P, _PP],
    "vyb_frame_encode": [_U, _P, C.c_size_t, _PP, C.POINTER(C.c_size_t)],
    "vyb_frame_decode": [_U, _P, C.c_size_t, _PP, C.POINTER(C.c_size_t), C.c_char_p],
    "vyb_payload_to_vtp0": [_P, C.c_char_p, _U, _P, _U, _PP, C.POINTER(C.c_size_t)],
    "vyb_payload_from_vtp0": [_P, C.c_size_t, _PP, C.c_char_p],
    "vyb_envelope_to_vme0": [_P, C.c_size_t, _P, _P, _U, _PP, C.POINTER(C.c_size_t)],
    "vyb_envelope_from_vme0": [_P, C.c_size_t, _U, _PP, C.POINTER(C.c_size_t), C.POINTER(C.c_uint32)],
    "vyb_unpack_i4x8_via": [_P, _P, C.c_size_t, _U, _P],
    "vyb_i4x8_dot_f32_scaled_via": [_P, _P, C.c_size_t, _P, C.c_size_t, C.c_float, C.c_float, _U, _P],
    "vyb_i4x8_matvec_f32_scaled_via": [_P, _P, C.c_size_t, _P, C.c_size_t, _P, C.c_size_t, _U, _U, _P],
    "vyb_i4x8_batched_matvec_f32_scaled_via": [_P, _P, C.c_size_t, _P, C.c_size_t, _P, C.c_size_t, _U, _U, _U, _P],
    "vyb_i4x8_batched_matmul_f32_scaled_via": [_P, _P, C.c_size_t, _P, C.c_size_t, _P, C.c_size_t, _P, C.c_size_t, _U, _U, _U, _P],
    "vyb_i4x8_batched_matmul_top1_f32_scaled_via": [_P, _P, C.c_size_t, _P, C.c_size_t, _P, C.c_size_t, _P, C.c_size_t, _U, _U, _U, _P, _P],
    "vyb_compile": [_P, _PP],
    "vyb_target_compile": [_P, _PP],
    "vyb_payload_bytes": [_P, C.POINTER(C.POINTER(C.c_uint8)), C.POINTER(C.c_size_t)],
    "vyb_payload_from_bytes": [C.c_char_p, C.c_size_t, _PP],
    "vyb_device_acquire": [C.c_int32, _PP],
    "vyb_device_identity_of": [_P, C.POINTER(DeviceIdentity)],
    "vyb_device_caps_of": [_P, C.POINTER(DeviceCaps)],
    "vyb_device_is_healthy": [_P],
    "vyb_device_mark_lost": [_P, _S],
    "vyb_device_reacquire": [_P],
    "vyb_alloc": [_P, C.c_size_t, C.POINTER(ResidentHandle)],
    "vyb_upload": [_P, ResidentHandle, _P, C.c_size_t],
    "vyb_upload_at": [_P, ResidentHandle, C.c_size_t, _P, C.c_size_t],
    "vyb_download": [_P, ResidentHandle, _P, C.c_size_t],
    "vyb_download_range": [_P, ResidentHandle, C.c_size_t, _P, C.c_size_t],
    "vyb_free": [_P, ResidentHandle],
    "vyb_resident_device_ptr": [_P, ResidentHandle, _PP, C.POINTER(C.c_size_t)],
    "vyb_materialize": [_P, _P, _P, _PP],
    "vyb_instance_device": [_P, C.POINTER(DeviceIdentity)],
    "vyb_submit": [_P, C.c_char_p, C.POINTER(Binding), C.c_size_t, C.POINTER(DispatchConfig), _PP],
    "vyb_prepare": [_P, C.c_char_p, C.POINTER(Binding), C.c_size_t, _PP],
    "vyb_prepared_submit": [_P, C.POINTER(Binding), C.c_size_t, _PP],
    "vyb_prepared_submit_after": [_P, _P, C.POINTER(Binding), C.c_size_t, _PP],
    "vyb_prepared_free": [_P],
    "vyb_instance_inject_status": [_P, _U],
    "vyb_submission_is_ready": [_P],
    "vyb_submission_wait": [_P, _PP],
    "vyb_completion_output": [_P, _U, C.POINTER(C.POINTER(C.c_uint8)), C.POINTER(C.c_size_t)],
    "vyb_completion_device_ns": [_P, C.POINTER(C.c_uint64)],
    "vyb_k_tensor_peak": [_U, _U, _P, _P, C.POINTER(C.c_double)],
    "vyb_k_colpar_push": [C.POINTER(AllGatherCtx), _P, _U, _U, C.c_uint64, C.c_uint64, _P, _P],
    "vyb_k_colpar_wait": [C.POINTER(AllGatherCtx), _U, _P, _P],
    "vyb_k_int4_gemv": [_P, _P, _P, _P, _U, _U, _U, _U, _U, _P, _P],
    "vyb_k_int4_gemv_ex": [_P, _P, _P, _P, _U, _U, _U, _U, _U, _U, _P, _P],
    "vyb_k_int4_linear_block": [_P, _P, C.c_float, _P, _P, _P, _P, _P, _U, _U, _U, _U, _U, _P, _P],
    "vyb_k_rms_norm": [_P, _P, _P, _U, _U, C.c_float, _U, _P],
    "vyb_k_residual_add": [_P, _P, _P, _U, _U, _P],
    "vyb_k_swiglu": [_P, _P, _P, _U, _U, _P],
    "vyb_k_int8_weight_only_linear": [_P, _P, _P, _P, _U, _U, _U, _P],
    "vyb_k_int4_prefill_gemm": [_P, _P, _P, _P, _U, _U, _U, _U, _U, _P, _P],
    "vyb_k_quantize_per_token_int8": [_P, _P, _P, _U, _U, _P],
    "vyb_k_int8_gemm_i32": [_P, _P, _P, _U, _U, _U, _P, _P],
    "vyb_k_int8_gemm_i32_ex": [_P, _P, _P, _U, _U, _U, _U, _P, _P],
    "vyb_k_allgather_push": [_P, _U, _U, _U, _P, _P],
    "vyb_k_allgather_wait": [_P, _P, _P],
    "vyb_k_int8_gemm_i32_gather": [_P, _P, _P, _U, _U, _U, C.c_uint64, C.c_uint64, _P, _P],
    "vyb_k_int4_gemv_allgather": [_P, _U, _P, _P, _P, _U, _U, _U, _U, _U, _P, _P],
    "vyb_k_moe_route": [_P, _P, _P, _P, _U, _U, _U, _U, _P],
    "vyb_k_rows_gather_bf16": [_P, _P, _P, _U, _U, _P],
    "vyb_k_moe_experts_int4": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _U, _U, _U, _U, _U, _P, _P],
    "vyb_k_moe_combine": [_P, _P, _P, _P, _U, _U, _U, _P],
    "vyb_k_moe_ep_sizes": [_U, _U, _U, _U, _U, _U, _U, _P, _P, _P],
    "vyb_k_moe_ep_ffn_int4": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _U, _U, _U, _U, _U, _U, _U, _P, _P],
    "vyb_k_moe_ffn_int4_scratch_bytes": [_U, _U, _U, _U, _U, _P],
    "vyb_k_moe_ffn_int4": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, C.c_uint64, _U, _U, _U, _U, _U, _U, _P, _P],
    "vyb_k_linear_int8_dynamic_static_scratch": [_P, _P, _P, _P, _U, _U, _U, _P, _P],
}

_OTHER_FUNCS = {
    "vyb_abi_version": (C.c_uint32, []),
    "vyb_last_error_message": (C.c_char_p, []),
    "vyb_supported_op_count": (C.c_uint32, []),
    "vyb_supported_op": (C.c_char_p, [_U]),
    "vyb_blake3": (None, [_P, C.c_size_t, C.c_char_p]),
    "vyb_i4_packed_words": (C.c_uint32, [_U]),
    "vyb_quantized_linear_4bit_spec_affine_grouped": (None, [_U, _U, _U, C.POINTER(QuantizedLinear4BitSpec)]),
    "vyb_program_op_id": (C.c_char_p, [_P]),
    "vyb_program_buffer_count": (C.c_uint32, [_P]),
    "vyb_program_workgroup_size": (None, [_P, C.POINTER(C.c_uint32 * 3)]),
    "vyb_program_is_trap": (C.c_uint32, [_P]),
    "vyb_program_trap_message": (C.c_char_p, [_P]),
    "vyb_program_fingerprint": (None, [_P, C.c_char_p]),
    "vyb_program_free": (None, [_P]),
    "vyb_artifact_digest": (None, [_P, C.c_char_p]),
    "vyb_artifact_free": (None, [_P]),
    "vyb_payload_digest": (None, [_P, C.c_char_p]),
    "vyb_payload_neutral_artifact": (None, [_P, C.c_char_p]),
    "vyb_graph_free": (None, [_P]),
    "vyb_graph_node_count": (C.c_uint32, [_P]),
    "vyb_graph_value_count": (C.c_uint32, [_P]),
    "vyb_graph_digest": (None, [_P, C.c_char_p]),
    "vyb_safetensors_free": (None, [_P]),
    "vyb_safetensors_identity": (None, [_P, C.c_char_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "vyb_quantized_scratch_free": (None, [_P]),
    "vyb_frame_free": (None, [_P]),
    "vyb_device_retain": (None, [_P]),
    "vyb_quantized_scratch_stats": (None, [_P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "vyb_safetensors_count": (C.c_uint32, [_P]),
    "vyb_payload_format": (C.c_char_p, [_P]),
    "vyb_payload_kernel_variant": (C.c_uint32, [_P]),
    "vyb_payload_free": (None, [_P]),
    "vyb_device_release": (None, [_P]),
    "vyb_instance_artifact_digest": (None, [_P, C.c_char_p]),
    "vyb_instance_payload_digest": (None, [_P, C.c_char_p]),
    "vyb_instance_free": (None, [_P]),
    "vyb_completion_output_count": (C.c_uint32, [_P]),
    "vyb_completion_free": (None, [_P]),
}


def exported_names() -> list[str]:
    return sorted(list(_STATUS_FUNCS) + list(_OTHER_FUNCS))


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m vyre_b200.build` (nvcc, sm_100a). "
                "The native library is the only implementation; there is no fallback.")
        L = C.CDLL(LIB_PATH)
        for name, args in _STATUS_FUNCS.items():
            fn = getattr(L, name)
            fn.restype = C.c_int32
            fn.argtypes = args
        for name, (res, args) in _OTHER_FUNCS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = lib().vyb_last_error_message()
        raise BackendError(rc, msg.decode("utf-8", "replace") if msg else "")
