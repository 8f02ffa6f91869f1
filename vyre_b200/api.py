"""Host-side mirror of the reference's operator and submission interface over the C ABI.

Names follow the Rust API so that tests read like the reference's own:
  builders   vyre_libs::nn::{linear_4bit, linear_4bit_affine_grouped[_batched][_typed], ...},
             vyre_primitives::math::quantized::{unpack_i4x8, i4x8_*}, vyre_libs::quant::{int8_*, int4_*}
  lifecycle  ProgramGraph -> Artifact (compile) -> TargetPayload (TargetCompiler) -> ArtifactInstance
             (ArtifactMaterializer) -> BindingSet -> Submission -> Completion, and ArtifactSession
             (vyre-runtime/src/artifact_admission.rs:152-496) tying them together.
Every call goes through libvyre_b200.so; nothing here computes.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

import numpy as np

from . import ffi
from .ffi import BackendError, check  # noqa: F401  (re-exported)


def _b(s: str) -> bytes:
    return s.encode()


class Program:
    """vyre_foundation::ir::Program as the native facet sees it (buffers, workgroup size, op region id)."""

    def __init__(self, handle: int, owner=None):
        self._h = C.c_void_p(handle)
        self._owner = owner  # a graph that owns the program: keeps it alive, and the handle is not freed here

    def __del__(self):
        try:
            if self._h and self._owner is None:
                ffi.lib().vyb_program_free(self._h)
        except Exception:
            pass

    @property
    def op_id(self) -> str:
        return ffi.lib().vyb_program_op_id(self._h).decode()

    def buffers(self) -> list[dict]:
        L = ffi.lib()
        out = []
        for i in range(L.vyb_program_buffer_count(self._h)):
            d = ffi.BufferDecl()
            check(L.vyb_program_buffer(self._h, i, C.byref(d)))
            out.append(dict(name=d.name.decode(), binding=d.binding, access=d.access, dtype=d.dtype, count=d.count,
                            output_byte_range=(int(d.output_byte_begin), int(d.output_byte_end))
                            if d.has_output_byte_range else None))
        return out

    def workgroup_size(self) -> list[int]:
        arr = (C.c_uint32 * 3)()
        ffi.lib().vyb_program_workgroup_size(self._h, C.byref(arr))
        return list(arr)

    @property
    def is_trap(self) -> bool:
        return bool(ffi.lib().vyb_program_is_trap(self._h))

    @property
    def trap_message(self) -> str:
        return ffi.lib().vyb_program_trap_message(self._h).decode()

    def fingerprint(self) -> bytes:
        buf = C.create_string_buffer(32)
        ffi.lib().vyb_program_fingerprint(self._h, buf)
        return buf.raw


def _build(fn_name: str, *args) -> Program:
    out = C.c_void_p()
    conv = [_b(a) if isinstance(a, str) else a for a in args]
    check(getattr(ffi.lib(), fn_name)(*conv, C.byref(out)))
    return Program(out.value)


# ---- vyre_libs::nn / quant / vyre_primitives builders (argument order = the Rust builders') ---------------
def linear_4bit(x, w_packed, b, out, in_dim, out_dim):
    return _build("vyb_nn_linear_4bit", x, w_packed, b, out, in_dim, out_dim)


def linear_4bit_affine_grouped(x, w_packed, scale, zero_point, b, out, in_dim, out_dim, group_size):
    return _build("vyb_nn_linear_4bit_affine_grouped", x, w_packed, scale, zero_point, b, out, in_dim, out_dim,
                  group_size)


def linear_4bit_affine_grouped_batched(x, w_packed, scale, zero_point, b, out, in_dim, out_dim, group_size,
                                       batch_size):
    return _build("vyb_nn_linear_4bit_affine_grouped_batched", x, w_packed, scale, zero_point, b, out, in_dim,
                  out_dim, group_size, batch_size)


@dataclass
class QuantizedLinear4BitSpec:
    in_dim: int
    out_dim: int
    storage_dtype: int = ffi.DT_I4
    scale_group_size: int = 0
    zero_point_group_size: int = 0

    @staticmethod
    def affine_grouped(in_dim: int, out_dim: int, group_size: int) -> "QuantizedLinear4BitSpec":
        s = ffi.QuantizedLinear4BitSpec()
        ffi.lib().vyb_quantized_linear_4bit_spec_affine_grouped(in_dim, out_dim, group_size, C.byref(s))
        return QuantizedLinear4BitSpec(s.in_dim, s.out_dim, s.storage_dtype, s.scale_group_size,
                                       s.zero_point_group_size)

    def _c(self):
        return ffi.QuantizedLinear4BitSpec(self.in_dim, self.out_dim, self.storage_dtype, self.scale_group_size,
                                           self.zero_point_group_size)


def linear_4bit_affine_grouped_typed(spec, x, w_packed, scale, zero_point, b, out):
    c = spec._c()
    return _build("vyb_nn_linear_4bit_affine_grouped_typed", C.byref(c), x, w_packed, scale, zero_point, b, out)


def linear_4bit_affine_grouped_batched_typed(spec, batch_size, x, w_packed, scale, zero_point, b, out):
    c = spec._c()
    return _build("vyb_nn_linear_4bit_affine_grouped_batched_typed", C.byref(c), batch_size, x, w_packed, scale,
                  zero_point, b, out)


def linear_4bit_affine_grouped_planner_evidence(spec) -> dict:
    c = spec._c()
    ev = ffi.PlannerEvidence()
    check(ffi.lib().vyb_nn_linear_4bit_affine_grouped_planner_evidence(C.byref(c), C.byref(ev)))
    d = {}
    for name, _ in ffi.PlannerEvidence._fields_:
        v = getattr(ev, name)
        d[name] = v.decode() if isinstance(v, bytes) else v
    return d


def unpack_i4x8(packed_words, out_lanes, lane_count):
    return _build("vyb_math_unpack_i4x8", packed_words, out_lanes, lane_count)


def i4x8_dot_i32(lhs, rhs, out, lane_count, lib_op_id=False):
    return _build("vyb_math_i4x8_dot_i32", lhs, rhs, out, lane_count, int(lib_op_id))


def i4x8_dot_f32_scaled(lhs, rhs, lhs_scale, rhs_scale, out, lane_count, lib_op_id=False):
    return _build("vyb_math_i4x8_dot_f32_scaled", lhs, rhs, lhs_scale, rhs_scale, out, lane_count, int(lib_op_id))


def i4x8_matvec_f32_scaled(weights, x, row_scales, out, rows, cols, lib_op_id=False):
    return _build("vyb_math_i4x8_matvec_f32_scaled", weights, x, row_scales, out, rows, cols, int(lib_op_id))


def i4x8_batched_matvec_f32_scaled(weights, x, row_scales, out, batch, rows, cols, lib_op_id=False):
    return _build("vyb_math_i4x8_batched_matvec_f32_scaled", weights, x, row_scales, out, batch, rows, cols,
                  int(lib_op_id))


def i4x8_batched_matmul_f32_scaled(weights, acts, row_scales, batch_scales, out, batch, rows, cols, lib_op_id=False):
    return _build("vyb_math_i4x8_batched_matmul_f32_scaled", weights, acts, row_scales, batch_scales, out, batch,
                  rows, cols, int(lib_op_id))


def i4x8_batched_matmul_top1_f32_scaled(weights, acts, row_scales, batch_scales, out, batch, rows, cols,
                                        lib_op_id=False):
    return _build("vyb_math_i4x8_batched_matmul_top1_f32_scaled", weights, acts, row_scales, batch_scales, out,
                  batch, rows, cols, int(lib_op_id))


def int8_unpack(packed, scales, output, n, cols):
    return _build("vyb_quant_int8_unpack", packed, scales, output, n, cols)


def int8_pack(input_, output, n):
    return _build("vyb_quant_int8_pack", input_, output, n)


def linear_rows(x, w, b, out, rows, in_dim, out_dim):
    return _build("vyb_nn_linear_rows", x, w, b, out, rows, in_dim, out_dim)


def linear_rows_no_bias(x, w, out, rows, in_dim, out_dim):
    return _build("vyb_nn_linear_rows_no_bias", x, w, out, rows, in_dim, out_dim)


def linear_rows_no_bias_typed(x, w, out, rows, in_dim, out_dim, dtype):
    return _build("vyb_nn_linear_rows_no_bias_typed", x, w, out, rows, in_dim, out_dim, dtype)


def linear_rows_no_bias_out_in_typed(x, w, out, rows, in_dim, out_dim, dtype):
    return _build("vyb_nn_linear_rows_no_bias_out_in_typed", x, w, out, rows, in_dim, out_dim, dtype)


def matmul(a, b, out, m, k, n):
    return _build("vyb_math_matmul", a, b, out, m, k, n)


def matmul_bias(a, b, bias, out, m, k, n):
    return _build("vyb_math_matmul_bias", a, b, bias, out, m, k, n)


def matmul_bias_tiled(a, b, bias, out, m, k, n, tile):
    return _build("vyb_math_matmul_bias_tiled", a, b, bias, out, m, k, n, tile)


def linear(x, w, b, out, in_dim, out_dim):
    """vyre_libs::nn::linear: u32 `out[i] = sum_k x[k] * w[k, i] + b[i]` (tiled form from in_dim * out_dim >= 1024)."""
    return _build("vyb_nn_linear", x, w, b, out, in_dim, out_dim)


def linear_tiled(x, w, b, out, in_dim, out_dim, tile):
    return _build("vyb_nn_linear_tiled", x, w, b, out, in_dim, out_dim, tile)


def moe_gate(input_scores, output_indices, output_weights, num_experts, k):
    return _build("vyb_nn_moe_gate", input_scores, output_indices, output_weights, num_experts, k)


def softmax_top_k(scores, out_indices, out_weights, n, k):
    return _build("vyb_nn_softmax_top_k", scores, out_indices, out_weights, n, k)


def top_k(input_, output_indices, n, k):
    return _build("vyb_nn_top_k", input_, output_indices, n, k)


def swiglu(gate, up, output, n):
    return _build("vyb_nn_swiglu", gate, up, output, n)


def swiglu_typed(gate, up, output, n, dtype):
    return _build("vyb_nn_swiglu_typed", gate, up, output, n, dtype)


def residual_add(residual, branch, output, n):
    return _build("vyb_nn_residual_add", residual, branch, output, n)


def residual_add_typed(residual, branch, output, n, dtype):
    return _build("vyb_nn_residual_add_typed", residual, branch, output, n, dtype)


def learned_rms_norm(input, weight, output, rows, hidden, eps, dtype):  # noqa: A002 - the reference's argument name
    return _build("vyb_nn_learned_rms_norm", input, weight, output, rows, hidden, C.c_float(eps), dtype)


def gated_rms_norm(input, weight, gate, output, rows, hidden, eps, dtype):  # noqa: A002
    return _build("vyb_nn_gated_rms_norm", input, weight, gate, output, rows, hidden, C.c_float(eps), dtype)


def gated_rms_norm_with_weight_dtype(input, weight, gate, output, rows, hidden, eps, dtype, weight_dtype):  # noqa: A002
    return _build("vyb_nn_gated_rms_norm_with_weight_dtype", input, weight, gate, output, rows, hidden, C.c_float(eps), dtype,
                  weight_dtype)


def q4_k_unpack(packed, scales, mins, output, n):
    return _build("vyb_quant_q4_k_unpack", packed, scales, mins, output, n)


def q2_k_unpack(packed, scales, mins, output, n):
    return _build("vyb_quant_q2_k_unpack", packed, scales, mins, output, n)


def q4_k_linear(x, w_packed, w_scales, w_mins, b, out, in_dim, out_dim):
    return _build("vyb_quant_q4_k_linear", x, w_packed, w_scales, w_mins, b, out, in_dim, out_dim)


def q2_k_linear(x, w_packed, w_scales, w_mins, b, out, in_dim, out_dim):
    return _build("vyb_quant_q2_k_linear", x, w_packed, w_scales, w_mins, b, out, in_dim, out_dim)


def expert_mlp(x, w_gate, b_gate, w_up, b_up, w_down, b_down, out, in_dim, hidden_dim, out_dim):
    return _build("vyb_nn_expert_mlp", x, w_gate, b_gate, w_up, b_up, w_down, b_down, out, in_dim, hidden_dim,
                  out_dim)


def moe_layer_route_and_accumulate(x, w_router, b_router, expert_indices, expert_weights, expert_outputs, out,
                                   in_dim, num_experts, out_dim, k):
    return _build("vyb_nn_moe_layer_route_and_accumulate", x, w_router, b_router, expert_indices, expert_weights,
                  expert_outputs, out, in_dim, num_experts, out_dim, k)


def linear_int4_grouped_rowmajor(x, w_packed, scale, out, batch, in_dim, out_dim, group_size, out_dtype=ffi.DT_BF16):
    return _build("vyb_nn_linear_int4_grouped_rowmajor", x, w_packed, scale, out, batch, in_dim, out_dim, group_size,
                  out_dtype)


def linear_int4_block(x, norm_weight, w_packed, scale, residual, out, batch, in_dim, out_dim, group_size, norm_eps=0.0, gate=None):
    """The int4 row-major projection as one node with a learned RMSNorm in front (`norm_weight` named) and, behind it,
    SwiGLU(gate, projection) (`gate` named) or a residual add (`residual` named); pass None for the parts that are absent."""
    opt = lambda name: None if name is None else _b(name)  # noqa: E731
    return _build("vyb_nn_linear_int4_block", x, opt(norm_weight), w_packed, scale, opt(gate), opt(residual), out, batch, in_dim,
                  out_dim, group_size, C.c_float(norm_eps))


def linear_int8_weight_only(x, w, scale, out, batch, in_dim, out_dim):
    return _build("vyb_nn_linear_int8_weight_only", x, w, scale, out, batch, in_dim, out_dim)


def linear_int8_dynamic(x, w, x_scale, out, rows, in_dim, out_dim):
    return _build("vyb_nn_linear_int8_dynamic", x, w, x_scale, out, rows, in_dim, out_dim)


def moe_ffn_int4(x, w_router, w13, s13, w2, s2, out, routing_idx, routing_w, tokens, hidden, inter, experts, topk,
                 group_size):
    return _build("vyb_nn_moe_ffn_int4", x, w_router, w13, s13, w2, s2, out, routing_idx, routing_w, tokens, hidden,
                  inter, experts, topk, group_size)


def blake3(data: bytes) -> bytes:
    buf = C.create_string_buffer(32)
    ffi.lib().vyb_blake3(data, len(data), buf)
    return buf.raw


def registration() -> dict:
    r = ffi.RegistrationInfo()
    check(ffi.lib().vyb_registration(C.byref(r)))
    return dict(id=r.id.decode(), target_id=r.target_id.decode(), payload_format=r.payload_format.decode(),
                format_version=r.format_version, precedence=r.precedence,
                profile=dict(identity=r.profile.identity.decode(), generation=r.profile.generation,
                             max_workgroup_size=list(r.profile.max_workgroup_size),
                             max_invocations=r.profile.max_invocations,
                             max_dynamic_shared_bytes=r.profile.max_dynamic_shared_bytes,
                             subgroup_size=r.profile.subgroup_size))


def supported_ops() -> list[str]:
    L = ffi.lib()
    return [L.vyb_supported_op(i).decode() for i in range(L.vyb_supported_op_count())]


# ---- lifecycle ---------------------------------------------------------------------------------------------
class Artifact:
    def __init__(self, handle):
        self._h = C.c_void_p(handle)

    def __del__(self):
        try:
            ffi.lib().vyb_artifact_free(self._h)
        except Exception:
            pass

    def digest(self) -> bytes:
        buf = C.create_string_buffer(32)
        ffi.lib().vyb_artifact_digest(self._h, buf)
        return buf.raw


def compile(program: Program) -> Artifact:  # noqa: A001 - mirrors vyre_megakernel::compile
    out = C.c_void_p()
    check(ffi.lib().vyb_compile(program._h, C.byref(out)))
    return Artifact(out.value)


class TargetPayload:
    def __init__(self, handle):
        self._h = C.c_void_p(handle)

    def __del__(self):
        try:
            ffi.lib().vyb_payload_free(self._h)
        except Exception:
            pass

    def digest(self) -> bytes:
        buf = C.create_string_buffer(32)
        ffi.lib().vyb_payload_digest(self._h, buf)
        return buf.raw

    def neutral_artifact(self) -> bytes:
        buf = C.create_string_buffer(32)
        ffi.lib().vyb_payload_neutral_artifact(self._h, buf)
        return buf.raw

    def format(self) -> str:
        return ffi.lib().vyb_payload_format(self._h).decode()

    def kernel_variant(self) -> int:
        return int(ffi.lib().vyb_payload_kernel_variant(self._h))

    def to_bytes(self) -> bytes:
        p = C.POINTER(C.c_uint8)()
        n = C.c_size_t()
        check(ffi.lib().vyb_payload_bytes(self._h, C.byref(p), C.byref(n)))
        return C.string_at(p, n.value)

    @staticmethod
    def from_bytes(data: bytes) -> "TargetPayload":
        out = C.c_void_p()
        check(ffi.lib().vyb_payload_from_bytes(data, len(data), C.byref(out)))
        return TargetPayload(out.value)


def target_compile(artifact: Artifact) -> TargetPayload:
    out = C.c_void_p()
    check(ffi.lib().vyb_target_compile(artifact._h, C.byref(out)))
    return TargetPayload(out.value)


class Device:
    """vyre_driver Device + ArtifactMaterializer for one acquired generation."""

    def __init__(self, ordinal: int = 0):
        out = C.c_void_p()
        check(ffi.lib().vyb_device_acquire(ordinal, C.byref(out)))
        self._h = out

    @staticmethod
    def acquire(ordinal: int = 0) -> "Device":
        return Device(ordinal)

    def release(self):
        if self._h:
            ffi.lib().vyb_device_release(self._h)
            self._h = None

    def identity(self) -> dict:
        i = ffi.DeviceIdentity()
        check(ffi.lib().vyb_device_identity_of(self._h, C.byref(i)))
        return dict(backend=i.backend.decode(), device=i.device.decode(), generation=i.generation)

    def caps(self) -> dict:
        c = ffi.DeviceCaps()
        check(ffi.lib().vyb_device_caps_of(self._h, C.byref(c)))
        return {n: (getattr(c, n).decode() if n == "name" else getattr(c, n)) for n, _ in ffi.DeviceCaps._fields_}

    def is_healthy(self) -> bool:
        return bool(ffi.lib().vyb_device_is_healthy(self._h))

    def mark_lost(self, reason: str = "injected by test"):
        check(ffi.lib().vyb_device_mark_lost(self._h, _b(reason)))

    def reacquire(self):
        check(ffi.lib().vyb_device_reacquire(self._h))

    # resident buffers
    def allocate_resident(self, byte_len: int) -> ffi.ResidentHandle:
        h = ffi.ResidentHandle()
        check(ffi.lib().vyb_alloc(self._h, byte_len, C.byref(h)))
        return h

    def upload_resident(self, h, data) -> None:
        a = np.ascontiguousarray(data)
        check(ffi.lib().vyb_upload(self._h, h, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def upload_resident_at(self, h, offset: int, data) -> None:
        a = np.ascontiguousarray(data)
        check(ffi.lib().vyb_upload_at(self._h, h, offset, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def download_resident(self, h, nbytes: int, offset: int = 0) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        check(ffi.lib().vyb_download_range(self._h, h, offset, out.ctypes.data_as(C.c_void_p), nbytes))
        return out

    def free_resident(self, h) -> None:
        check(ffi.lib().vyb_free(self._h, h))

    def resident_ptr(self, h) -> tuple[int, int]:
        p = C.c_void_p()
        n = C.c_size_t()
        check(ffi.lib().vyb_resident_device_ptr(self._h, h, C.byref(p), C.byref(n)))
        return p.value, n.value

    def resident_from(self, data) -> ffi.ResidentHandle:
        a = np.ascontiguousarray(data)
        h = self.allocate_resident(a.nbytes)
        self.upload_resident(h, a)
        return h

    def materialize(self, artifact: Artifact, payload: TargetPayload) -> "ArtifactInstance":
        out = C.c_void_p()
        check(ffi.lib().vyb_materialize(self._h, artifact._h, payload._h, C.byref(out)))
        return ArtifactInstance(out.value, self)


def program_from_op(op_id: str, buffers: list[dict], op_spec: list[int] | None = None) -> Program:
    """Rebuilds a Program from what a vyre Artifact carries: the op id and the BufferDecls (dicts as Program.buffers()
    returns them), optionally the op's dimensions in builder order (vyb_program_from_op)."""
    arr = (ffi.BufferDecl * max(1, len(buffers)))()
    keep = []
    for i, b in enumerate(buffers):
        name = b["name"].encode()
        keep.append(name)
        arr[i].name, arr[i].binding, arr[i].access, arr[i].dtype, arr[i].count = name, b["binding"], b["access"], b["dtype"], b["count"]
        if b.get("output_byte_range"):
            arr[i].has_output_byte_range = 1
            arr[i].output_byte_begin, arr[i].output_byte_end = b["output_byte_range"]
    spec = (C.c_uint32 * max(1, len(op_spec or [])))(*(op_spec or []))
    out = C.c_void_p()
    check(ffi.lib().vyb_program_from_op(op_id.encode(), arr, len(buffers), spec if op_spec else None, len(op_spec or []), C.byref(out)))
    return Program(out.value)


class BindingSet:
    """vyre_driver BindingSet: values keyed by ArtifactValueId (= buffer binding slot)."""

    def __init__(self, artifact_digest: bytes):
        self.artifact = artifact_digest
        self.resources: dict[int, object] = {}
        self.invocation_grid = None
        self._marshalled = None

    def insert_host(self, value_id: int, data) -> None:
        self.resources[value_id] = np.ascontiguousarray(data)
        self._marshalled = None

    def insert_resident(self, value_id: int, handle) -> None:
        self.resources[value_id] = handle
        self._marshalled = None

    def marshal(self):
        """The C array of vyb_binding for this set (built once; a set that is submitted again and again - same
        buffers, new contents - costs no per-submit marshalling)."""
        if self._marshalled is None:
            arr = (ffi.Binding * max(1, len(self.resources)))()
            keep = []
            for i, (vid, res) in enumerate(sorted(self.resources.items())):
                arr[i].value_id = vid
                if isinstance(res, ffi.ResidentHandle):
                    arr[i].kind = ffi.BIND_RESIDENT
                    arr[i].resident = res
                else:
                    arr[i].kind = ffi.BIND_HOST
                    arr[i].host_ptr = res.ctypes.data
                    arr[i].len = res.nbytes
                    keep.append(res)
            self._marshalled = (arr, keep, len(self.resources))
        return self._marshalled

    def set_invocation_grid(self, grid) -> None:
        if any(g == 0 for g in grid):
            axis = [g == 0 for g in grid].index(True)
            raise BackendError(ffi.ERR_INVALID_PROGRAM,
                               f"Fix: invocation grid axis {axis} must be positive, got {grid[axis]}.")
        self.invocation_grid = list(grid)


class Completion:
    def __init__(self, handle):
        self._h = C.c_void_p(handle)

    def __del__(self):
        try:
            ffi.lib().vyb_completion_free(self._h)
        except Exception:
            pass

    def output(self, value_id: int) -> bytes:
        p = C.POINTER(C.c_uint8)()
        n = C.c_size_t()
        check(ffi.lib().vyb_completion_output(self._h, value_id, C.byref(p), C.byref(n)))
        return C.string_at(p, n.value)

    def output_view(self, value_id: int, dtype) -> np.ndarray:
        """Zero-copy view of the pinned readback buffer; valid until this Completion is dropped."""
        p = C.POINTER(C.c_uint8)()
        n = C.c_size_t()
        check(ffi.lib().vyb_completion_output(self._h, value_id, C.byref(p), C.byref(n)))
        return np.ctypeslib.as_array(p, shape=(n.value,)).view(dtype)

    @property
    def device_ns(self):
        ns = C.c_uint64()
        rc = ffi.lib().vyb_completion_device_ns(self._h, C.byref(ns))
        return ns.value if rc == 0 else None


class Submission:
    def __init__(self, handle, keepalive):
        self._h = C.c_void_p(handle)
        self._keep = keepalive

    def is_ready(self) -> bool:
        return bool(ffi.lib().vyb_submission_is_ready(self._h))

    def wait(self) -> Completion:
        out = C.c_void_p()
        h, self._h = self._h, None
        if h is None:
            raise BackendError(ffi.ERR_INVALID_PROGRAM, "Fix: completion may be consumed only once.")
        check(ffi.lib().vyb_submission_wait(h, C.byref(out)))
        self._keep = None
        return Completion(out.value)


class ArtifactInstance:
    def __init__(self, handle, device: Device):
        self._h = C.c_void_p(handle)
        self._dev = device

    def __del__(self):
        try:
            ffi.lib().vyb_instance_free(self._h)
        except Exception:
            pass

    def artifact(self) -> bytes:
        buf = C.create_string_buffer(32)
        ffi.lib().vyb_instance_artifact_digest(self._h, buf)
        return buf.raw

    def payload(self) -> bytes:
        buf = C.create_string_buffer(32)
        ffi.lib().vyb_instance_payload_digest(self._h, buf)
        return buf.raw

    def device(self) -> dict:
        i = ffi.DeviceIdentity()
        check(ffi.lib().vyb_instance_device(self._h, C.byref(i)))
        return dict(backend=i.backend.decode(), device=i.device.decode(), generation=i.generation)

    def submit(self, bindings: BindingSet, leave_resident: bool = False, config: ffi.DispatchConfig | None = None):
        arr, keep, count = bindings.marshal()
        cfg = config or ffi.DispatchConfig()
        if bindings.invocation_grid:
            for a in range(3):
                cfg.grid_override[a] = bindings.invocation_grid[a]
        if leave_resident:
            cfg.leave_resident = 1
        out = C.c_void_p()
        check(ffi.lib().vyb_submit(self._h, bindings.artifact, arr, count, C.byref(cfg),
                                   C.byref(out)))
        return Submission(out.value, keep)


class PreparedSubmission:
    """A binding set validated once and frozen into one device-side graph (vyb_prepare): a submission is then a copy of
    the changed host inputs plus a single graph launch. One submission per prepared set may be in flight."""

    def __init__(self, instance: ArtifactInstance, bindings: BindingSet):
        arr, keep, count = bindings.marshal()
        out = C.c_void_p()
        check(ffi.lib().vyb_prepare(instance._h, bindings.artifact, arr, count, C.byref(out)))
        self._h = C.c_void_p(out.value)
        self._instance = instance
        self._updates: dict[tuple, tuple] = {}

    def submit(self, host_inputs: dict | None = None, after: "Submission | None" = None) -> Submission:
        """host_inputs: {value_id: array} for the host-bound inputs whose bytes changed (copied in here). `after`: a pending
        submission (of any instance on the device) behind which this one is ordered on the device."""
        items = sorted((host_inputs or {}).items())
        key = tuple((vid, a.ctypes.data, a.nbytes) for vid, a in items)
        if key not in self._updates:  # same arrays again and again: marshalled once
            arr = (ffi.Binding * max(1, len(items)))()
            for i, (vid, a) in enumerate(items):
                if not a.flags["C_CONTIGUOUS"]:
                    raise BackendError(ffi.ERR_INVALID_PROGRAM, "Fix: pass C-contiguous arrays to a prepared submission.")
                arr[i].value_id, arr[i].kind, arr[i].host_ptr, arr[i].len = vid, ffi.BIND_HOST, a.ctypes.data, a.nbytes
            self._updates = {key: (arr, [a for _, a in items], len(items))}
        arr, keep, count = self._updates[key]
        out = C.c_void_p()
        if after is not None and after._h is None:
            raise BackendError(ffi.ERR_INVALID_PROGRAM, "Fix: `after` has been waited for already; order behind a pending submission.")
        check(ffi.lib().vyb_prepared_submit_after(self._h, after._h if after is not None else None, arr, count, C.byref(out)))
        return Submission(out.value, keep)

    def free(self) -> None:
        if self._h is not None:
            h, self._h = self._h, None
            check(ffi.lib().vyb_prepared_free(h))

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class ArtifactSession:
    """vyre_runtime::ArtifactSession: compile -> attach target -> materialize -> submit
    (vyre-runtime/src/artifact_admission.rs:152-496)."""

    def __init__(self, program: Program, device: Device, envelope: bytes | None = None):
        self.program = program
        self.device = device
        self.artifact = compile(program)
        self.payload = TargetPayload.from_bytes(envelope) if envelope is not None else target_compile(self.artifact)
        self.instance = device.materialize(self.artifact, self.payload)
        self._buffers = program.buffers()

    @staticmethod
    def compile(program: Program, device: Device) -> "ArtifactSession":
        return ArtifactSession(program, device)

    def envelope_bytes(self) -> bytes:
        return self.payload.to_bytes()

    def kernel_variant(self) -> int:
        """The hand-written kernel the target compiler chose for this program (0: reference evaluation order)."""
        return self.payload.kernel_variant()

    def rematerialize(self) -> None:
        """Re-admit the same authenticated payload bytes on the device's current generation; never recompiles
        (artifact_admission.rs:271-291)."""
        self.instance = self.device.materialize(self.artifact, TargetPayload.from_bytes(self.payload.to_bytes()))

    def input_slots(self) -> list[dict]:
        return [b for b in self._buffers if b["access"] in (ffi.ACCESS_READ_ONLY, ffi.ACCESS_READ_WRITE)]

    def output_slots(self) -> list[dict]:
        return [b for b in self._buffers if b["access"] in (ffi.ACCESS_OUTPUT, ffi.ACCESS_READ_WRITE)]

    def host_bindings(self, inputs: list) -> BindingSet:
        """Inputs in ABI slot order of the ReadOnly / ReadWrite values (artifact_admission.rs:398-434)."""
        slots = self.input_slots()
        if len(inputs) != len(slots):
            raise BackendError(ffi.ERR_INVALID_PROGRAM,
                               f"Fix: expected {len(slots)} host input(s) in slot order, got {len(inputs)}.")
        bs = BindingSet(self.artifact.digest())
        for slot, data in zip(slots, inputs):
            bs.insert_host(slot["binding"], data)
        return bs

    def submit(self, bindings: BindingSet, **kw) -> Submission:
        return self.instance.submit(bindings, **kw)

    def prepare(self, bindings: BindingSet) -> PreparedSubmission:
        return PreparedSubmission(self.instance, bindings)

    def submit_and_wait(self, bindings: BindingSet, **kw) -> Completion:
        return self.instance.submit(bindings, **kw).wait()

    def ordered_outputs(self, completion: Completion) -> list[bytes]:
        """Writable values in slot order (artifact_admission.rs:442-480)."""
        return [completion.output(b["binding"]) for b in self.output_slots()]

    def run_host(self, inputs: list) -> list[bytes]:
        c = self.submit_and_wait(self.host_bindings(inputs))
        return self.ordered_outputs(c)


# ---- safetensors ingestion (vyre-safetensors/src/lib.rs:108-260) --------------------------------------------------------
class SafetensorIndex:
    """vyre_safetensors::SafetensorIndex: the validated metadata of one shard; tensor bytes go straight from the file
    into resident device buffers (`load_resident`), where they bind as `Constant` values."""

    def __init__(self, handle, path: str):
        self._h = C.c_void_p(handle)
        self.path = path

    @staticmethod
    def open(path: str) -> "SafetensorIndex":
        out = C.c_void_p()
        check(ffi.lib().vyb_safetensors_open(os.fsencode(path), C.byref(out)))
        return SafetensorIndex(out.value, path)

    def __del__(self):
        try:
            if self._h:
                ffi.lib().vyb_safetensors_free(self._h)
                self._h = None
        except Exception:
            pass

    def identity(self) -> dict:
        """SafetensorShardIdentity: BLAKE3 of the exact header bytes, file length, payload start."""
        digest = C.create_string_buffer(32)
        flen, start = C.c_uint64(), C.c_uint64()
        ffi.lib().vyb_safetensors_identity(self._h, digest, C.byref(flen), C.byref(start))
        return {"header_digest": digest.raw, "file_len": flen.value, "data_start": start.value}

    def _entry(self, index: int) -> dict:
        e = ffi.SafetensorEntry()
        check(ffi.lib().vyb_safetensors_entry(self._h, index, C.byref(e)))
        return {"name": e.name.decode(), "dtype": e.dtype_name.decode(), "shape": [e.shape[i] for i in range(e.rank)],
                "file_range": (e.file_begin, e.file_end), "index": index}

    def tensors(self) -> list[dict]:
        """Tensors in canonical name order."""
        return [self._entry(i) for i in range(ffi.lib().vyb_safetensors_count(self._h))]

    def tensor(self, name: str) -> dict:
        idx = C.c_uint32()
        check(ffi.lib().vyb_safetensors_find(self._h, name.encode(), C.byref(idx)))
        return self._entry(idx.value)

    def require(self, name: str, dtype: str, shape) -> dict:
        """SafetensorRequirement: the tensor must be stored with exactly this dtype and shape."""
        arr = (C.c_uint64 * max(1, len(shape)))(*shape)
        idx = C.c_uint32()
        check(ffi.lib().vyb_safetensors_require(self._h, name.encode(), dtype.encode(), arr, len(shape), C.byref(idx)))
        return self._entry(idx.value)

    def load_resident(self, device: "Device", name: str, handle=None, offset: int = 0):
        """Allocate a resident buffer of the tensor's size (unless `handle` is given) and fill it from the file."""
        e = self.tensor(name)
        nbytes = e["file_range"][1] - e["file_range"][0]
        h = handle if handle is not None else device.allocate_resident(max(nbytes, 1))
        check(ffi.lib().vyb_safetensors_upload(self._h, e["index"], device._h, h, offset))
        return h


# ---- ProgramGraph (vyre-foundation/src/ir_inner/model/program_graph.rs) ---------------------------------------------------
_DT_SIZE = {ffi.DT_U32: 4, ffi.DT_I32: 4, ffi.DT_F16: 2, ffi.DT_BF16: 2, ffi.DT_F32: 4, ffi.DT_U8: 1, ffi.DT_I8: 1}


def value_contract(dtype: int, shape, lifetime: int, access: int = ffi.ACCESS_READ_ONLY) -> ffi.ValueContract:
    """ValueContract { dtype, shape, access, lifetime } (program_graph.rs:44-56); dimensions are statically known."""
    c = ffi.ValueContract()
    c.dtype, c.access, c.lifetime, c.rank = dtype, access, lifetime, len(shape)
    if len(shape) > 6:
        raise BackendError(ffi.ERR_INVALID_PROGRAM, "Fix: a value contract holds at most six dimensions.")
    for i, d in enumerate(shape):
        c.shape[i] = d
    return c


def _contract_dict(c: ffi.ValueContract) -> dict:
    return {"dtype": c.dtype, "access": c.access, "lifetime": c.lifetime, "shape": [int(c.shape[i]) for i in range(c.rank)]}


class ProgramGraph:
    """vyre_foundation::ir::ProgramGraph: Programs connected by typed values; construction order is the schedule."""

    def __init__(self, handle=None):
        if handle is None:
            out = C.c_void_p()
            check(ffi.lib().vyb_graph_new(C.byref(out)))
            handle = out.value
        self._h = C.c_void_p(handle)

    def __del__(self):
        try:
            if self._h:
                ffi.lib().vyb_graph_free(self._h)
                self._h = None
        except Exception:
            pass

    @staticmethod
    def from_program(node_name: str, program: Program) -> "ProgramGraph":
        out = C.c_void_p()
        check(ffi.lib().vyb_graph_from_program(node_name.encode(), program._h, C.byref(out)))
        return ProgramGraph(out.value)

    def add_external_value(self, name: str, contract: ffi.ValueContract) -> int:
        vid = C.c_uint32()
        check(ffi.lib().vyb_graph_add_external_value(self._h, name.encode(), C.byref(contract), C.byref(vid)))
        return vid.value

    def add_node(self, name: str, program: Program, inputs: list, outputs: list):
        """inputs: [(buffer, value id, contract)], outputs: [(buffer, value name, contract[, retained_successor_of])].
        Returns (node id, [output value ids])."""
        ins = (ffi.GraphInput * max(1, len(inputs)))()
        keep = []
        for i, (buf, val, con) in enumerate(inputs):
            b = buf.encode()
            keep.append(b)
            ins[i].buffer, ins[i].value, ins[i].contract = b, val, con
        outs = (ffi.GraphOutput * max(1, len(outputs)))()
        for i, o in enumerate(outputs):
            b, n = o[0].encode(), o[1].encode()
            keep += [b, n]
            outs[i].buffer, outs[i].name, outs[i].contract = b, n, o[2]
            outs[i].retained_successor_of = o[3] if len(o) > 3 and o[3] is not None else -1
        nid = C.c_uint32()
        vids = (C.c_uint32 * max(1, len(outputs)))()
        check(ffi.lib().vyb_graph_add_node(self._h, name.encode(), program._h, ins, len(inputs), outs, len(outputs), C.byref(nid), vids))
        return nid.value, [vids[i] for i in range(len(outputs))]

    def values(self) -> list[dict]:
        L, out = ffi.lib(), []
        for i in range(L.vyb_graph_value_count(self._h)):
            v = ffi.GraphValueInfo()
            check(L.vyb_graph_value(self._h, i, C.byref(v)))
            out.append({"id": i, "name": v.name.decode(), "contract": _contract_dict(v.contract),
                        "producer": None if v.producer < 0 else int(v.producer), "consumers": v.n_consumers,
                        "retained_successor_of": None if v.retained_successor_of < 0 else int(v.retained_successor_of),
                        "live": (v.live_start, v.live_end)})
        return out

    def nodes(self) -> list[dict]:
        L, out = ffi.lib(), []
        for i in range(L.vyb_graph_node_count(self._h)):
            n = ffi.GraphNodeInfo()
            check(L.vyb_graph_node(self._h, i, C.byref(n)))
            ins, outs = [], []
            for k in range(n.n_inputs):
                p = ffi.GraphInput()
                check(L.vyb_graph_node_input(self._h, i, k, C.byref(p)))
                ins.append({"buffer": p.buffer.decode(), "value": p.value, "contract": _contract_dict(p.contract)})
            for k in range(n.n_outputs):
                p, vid = ffi.GraphOutput(), C.c_uint32()
                check(L.vyb_graph_node_output(self._h, i, k, C.byref(p), C.byref(vid)))
                outs.append({"buffer": p.buffer.decode(), "name": p.name.decode(), "value": vid.value, "contract": _contract_dict(p.contract)})
            out.append({"id": i, "name": n.name.decode(), "program": Program(n.program, owner=self), "inputs": ins, "outputs": outs})
        return out

    def schedule(self) -> list[int]:
        return list(range(ffi.lib().vyb_graph_node_count(self._h)))

    def fuse_linear_blocks(self) -> tuple["ProgramGraph", int]:
        """A copy in which RMSNorm nodes in front of int4 linears and residual adds behind them are taken into
        `linear_int4_block` nodes wherever the decode kernel does the part in its own launch; (graph, nodes taken in)."""
        out, n = C.c_void_p(), C.c_uint32()
        check(ffi.lib().vyb_graph_fuse_linear_blocks(self._h, C.byref(out), C.byref(n)))
        return ProgramGraph(out.value), n.value

    def digest(self) -> bytes:
        buf = C.create_string_buffer(32)
        ffi.lib().vyb_graph_digest(self._h, buf)
        return buf.raw


class GraphSession:
    """Runs a ProgramGraph on a device: one materialised artifact per node, every value a resident buffer. `Constant`
    external values are uploaded once (`set_constant`, or a resident handle from `SafetensorIndex.load_resident`);
    `Invocation` external values are uploaded per run; produced values stay on the device between nodes; `Output`
    values are read back at the end of `run`."""

    def __init__(self, graph: ProgramGraph, device: "Device"):
        self.graph, self.device = graph, device
        self.values, self.nodes = graph.values(), graph.nodes()
        self.sessions = [ArtifactSession.compile(n["program"], device) for n in self.nodes]
        self.handles: dict[int, object] = {}
        self._owned: list = []
        self._chain = None  # run_chained: one prepared binding set per node
        for v in self.values:
            if v["producer"] is not None or v["contract"]["lifetime"] == ffi.LIFETIME_INVOCATION:
                self.handles[v["id"]] = self._alloc(v)

    def _bytes(self, v: dict) -> int:
        n = 1
        for d in v["contract"]["shape"]:
            n *= d
        return max(1, n * _DT_SIZE[v["contract"]["dtype"]])

    def _alloc(self, v: dict):
        h = self.device.allocate_resident(self._bytes(v))
        self._owned.append(h)
        return h

    def _by_name(self, name: str) -> dict:
        for v in self.values:
            if v["name"] == name:
                return v
        raise BackendError(ffi.ERR_INVALID_PROGRAM, f"Fix: the graph has no value named `{name}`.")

    def set_constant(self, name: str, data=None, handle=None) -> None:
        v = self._by_name(name)
        if v["producer"] is not None or v["contract"]["lifetime"] not in (ffi.LIFETIME_CONSTANT, ffi.LIFETIME_RETAINED):
            raise BackendError(ffi.ERR_INVALID_PROGRAM, f"Fix: `{name}` is not an external Constant or Retained value.")
        if handle is None:
            a = np.ascontiguousarray(data)
            if a.nbytes != self._bytes(v):
                raise BackendError(ffi.ERR_INVALID_PROGRAM,
                                   f"Fix: constant `{name}` needs {self._bytes(v)} bytes by its contract, got {a.nbytes}.")
            handle = self.device.resident_from(a)
            self._owned.append(handle)
        self._drop_chain()  # prepared sets have the old buffer's address baked in
        self.handles[v["id"]] = handle

    def run(self, inputs: dict) -> dict:
        """inputs: {external Invocation value name: array}. Returns {Output value name: bytes}."""
        for v in self.values:
            if v["producer"] is None and v["contract"]["lifetime"] == ffi.LIFETIME_INVOCATION:
                if v["name"] not in inputs:
                    raise BackendError(ffi.ERR_INVALID_PROGRAM, f"Fix: bind the graph input `{v['name']}`.")
                a = np.ascontiguousarray(inputs[v["name"]])
                if a.nbytes != self._bytes(v):
                    raise BackendError(ffi.ERR_INVALID_PROGRAM,
                                       f"Fix: graph input `{v['name']}` needs {self._bytes(v)} bytes by its contract, got {a.nbytes}.")
                self.device.upload_resident(self.handles[v["id"]], a)
            elif v["producer"] is None and v["id"] not in self.handles:
                raise BackendError(ffi.ERR_INVALID_PROGRAM, f"Fix: set the constant `{v['name']}` before running the graph.")
        for node, sess in zip(self.nodes, self.sessions):
            slot = {b["name"]: b["binding"] for b in sess._buffers}
            bs = BindingSet(sess.artifact.digest())
            for port in node["inputs"] + node["outputs"]:
                bs.insert_resident(slot[port["buffer"]], self.handles[port["value"]])
            done = sess.submit(bs, leave_resident=True).wait()
            del done
        out = {}
        for v in self.values:
            if v["contract"]["lifetime"] == ffi.LIFETIME_OUTPUT:
                out[v["name"]] = self.device.download_resident(self.handles[v["id"]], self._bytes(v)).tobytes()
        return out

    def _is_input(self, v: dict) -> bool:
        return v["producer"] is None and v["contract"]["lifetime"] == ffi.LIFETIME_INVOCATION

    def _drop_chain(self) -> None:
        if self._chain:
            for prep, _, _ in self._chain:
                prep.free()
        self._chain = None

    def run_chained(self, inputs: dict) -> dict:
        """The same as `run`, without the host in between: every node is a prepared binding set (graph inputs bound as host
        bytes of the nodes that read them, all other values resident, `Output` values that nothing reads handed back by the
        node's completion), submitted back to back in schedule order, each ordered on the device behind the one before;
        the host waits once the last node is submitted."""
        arrays = {}
        for v in self.values:
            if self._is_input(v):
                if v["name"] not in inputs:
                    raise BackendError(ffi.ERR_INVALID_PROGRAM, f"Fix: bind the graph input `{v['name']}`.")
                a = np.ascontiguousarray(inputs[v["name"]])
                if a.nbytes != self._bytes(v):
                    raise BackendError(ffi.ERR_INVALID_PROGRAM,
                                       f"Fix: graph input `{v['name']}` needs {self._bytes(v)} bytes by its contract, got {a.nbytes}.")
                arrays[v["name"]] = a
            elif v["producer"] is None and v["id"] not in self.handles:
                raise BackendError(ffi.ERR_INVALID_PROGRAM, f"Fix: set the constant `{v['name']}` before running the graph.")
        if self._chain is None:
            chain = []
            for node, sess in zip(self.nodes, self.sessions):
                slot = {b["name"]: b["binding"] for b in sess._buffers}
                bs, host, outs = BindingSet(sess.artifact.digest()), {}, {}
                for port in node["inputs"]:
                    v = self.values[port["value"]]
                    if self._is_input(v):
                        bs.insert_host(slot[port["buffer"]], arrays[v["name"]])
                        host[slot[port["buffer"]]] = v["name"]
                    else:
                        bs.insert_resident(slot[port["buffer"]], self.handles[port["value"]])
                for port in node["outputs"]:
                    v = self.values[port["value"]]
                    if v["contract"]["lifetime"] == ffi.LIFETIME_OUTPUT and v["consumers"] == 0:
                        outs[slot[port["buffer"]]] = v["name"]  # allocated by the backend, read from the completion
                    else:
                        bs.insert_resident(slot[port["buffer"]], self.handles[port["value"]])
                chain.append((sess.prepare(bs), host, outs))
            self._chain = chain
        subs, prev = [], None
        for prep, host, _ in self._chain:
            prev = prep.submit({s: arrays[name] for s, name in host.items()}, after=prev)
            subs.append(prev)
        out, failure = {}, None
        for sub, (_, _, outs) in zip(subs, self._chain):
            try:
                done = sub.wait()
                for s, name in outs.items():
                    out[name] = done.output(s)
                del done
            except BackendError as e:  # every submission is waited for, the first failure is reported
                failure = failure or e
        if failure:
            raise failure
        for v in self.values:
            if v["contract"]["lifetime"] == ffi.LIFETIME_OUTPUT and v["name"] not in out:
                out[v["name"]] = self.device.download_resident(self.handles[v["id"]], self._bytes(v)).tobytes()
        return out

    def close(self) -> None:
        self._drop_chain()
        for h in self._owned:
            try:
                self.device.free_resident(h)
            except Exception:
                pass
        self._owned = []


@dataclass
class QuantizedGatedMlpSpec:
    """Dimensions of a gated MLP with int4 group-quantized projections (the serving-layout form of
    vyre_libs::nn::model::DenseGatedMlpSpec, dense_gated_mlp.rs:15-29): bf16 activations, row-major packed weights."""
    rows: int
    hidden_dim: int
    intermediate_dim: int
    group_size: int = 128
    norm_eps: float | None = None  # a value makes the graph the whole residual block: RMSNorm in front, residual add behind


def quantized_gated_mlp_graph(spec: QuantizedGatedMlpSpec) -> ProgramGraph:
    """gate_proj and up_proj (int4 weights, `Constant`), SwiGLU, down_proj: vyre_libs::nn::model::dense_gated_mlp_graph
    (dense_gated_mlp.rs:59-370) over this backend's quantized linears, with the same value names. Without `norm_eps` the
    graph is the projection / activation / projection part (input `mlp.normalized`, output `mlp.down`); with it the graph
    is the reference's whole block: `residual` -> learned RMSNorm (bf16, `post_attention_layernorm.weight`) -> projections
    -> residual add -> `mlp.block_output`."""
    r, h, i, g = spec.rows, spec.hidden_dim, spec.intermediate_dim, spec.group_size
    if min(r, h, i, g) <= 0:
        raise BackendError(ffi.ERR_INVALID_PROGRAM, "Fix: rows, hidden_dim, intermediate_dim and group_size must be nonzero.")
    bf16 = ffi.DT_BF16
    inv, const, outl = ffi.LIFETIME_INVOCATION, ffi.LIFETIME_CONSTANT, ffi.LIFETIME_OUTPUT
    ro, rw = ffi.ACCESS_READ_ONLY, ffi.ACCESS_READ_WRITE
    read_hidden = value_contract(bf16, [r, h], inv, ro)
    read_inter, write_inter = value_contract(bf16, [r, i], inv, ro), value_contract(bf16, [r, i], inv, rw)
    # packed weights are declared as 32-bit words of eight nibbles (vyre-primitives/src/math/quantized/programs.rs:217-225)
    up_w, up_s = value_contract(ffi.DT_U32, [i, h // 8], const), value_contract(bf16, [i, h // g], const)
    down_w, down_s = value_contract(ffi.DT_U32, [h, i // 8], const), value_contract(bf16, [h, i // g], const)
    graph = ProgramGraph()
    whole = spec.norm_eps is not None
    write_hidden = value_contract(bf16, [r, h], inv, rw)
    if whole:
        residual = graph.add_external_value("residual", read_hidden)
        norm_c = value_contract(bf16, [h], const)
        norm_w = graph.add_external_value("post_attention_layernorm.weight", norm_c)
        _, (x,) = graph.add_node("mlp.norm", learned_rms_norm("input", "weight", "output", r, h, spec.norm_eps, bf16),
                                 [("input", residual, read_hidden), ("weight", norm_w, norm_c)], [("output", "mlp.normalized", write_hidden)])
    else:
        x = graph.add_external_value("mlp.normalized", read_hidden)
    gw = graph.add_external_value("mlp.gate_proj.qweight", up_w)
    gs = graph.add_external_value("mlp.gate_proj.scales", up_s)
    uw = graph.add_external_value("mlp.up_proj.qweight", up_w)
    us = graph.add_external_value("mlp.up_proj.scales", up_s)
    dw = graph.add_external_value("mlp.down_proj.qweight", down_w)
    ds = graph.add_external_value("mlp.down_proj.scales", down_s)

    def proj(name, out_name, inp, inp_contract, w, wc, s, sc, k, n, out_contract):
        prog = linear_int4_grouped_rowmajor("input", "weight", "scale", "output", r, k, n, g, bf16)
        _, (val,) = graph.add_node(name, prog, [("input", inp, inp_contract), ("weight", w, wc), ("scale", s, sc)],
                                   [("output", out_name, out_contract)])
        return val

    gate = proj("mlp.gate_proj", "mlp.gate", x, read_hidden, gw, up_w, gs, up_s, h, i, write_inter)
    up = proj("mlp.up_proj", "mlp.up", x, read_hidden, uw, up_w, us, up_s, h, i, write_inter)
    _, (act,) = graph.add_node("mlp.swiglu", swiglu_typed("gate", "up", "output", r * i, bf16),
                               [("gate", gate, read_inter), ("up", up, read_inter)], [("output", "mlp.activated", write_inter)])
    down = proj("mlp.down_proj", "mlp.down", act, read_inter, dw, down_w, ds, down_s, i, h,
                write_hidden if whole else value_contract(bf16, [r, h], outl, rw))
    if whole:
        graph.add_node("mlp.residual", residual_add_typed("residual", "branch", "output", r * h, bf16),
                       [("residual", residual, read_hidden), ("branch", down, read_hidden)],
                       [("output", "mlp.block_output", value_contract(bf16, [r, h], outl, rw))])
    return graph


@dataclass
class DenseGatedMlpSpec:
    """vyre_libs::nn::model::DenseGatedMlpSpec (dense_gated_mlp.rs:15-29): batch x sequence token rows, the RMSNorm epsilon,
    F16 / BF16 / F32 activations and weights."""
    batch: int
    sequence: int
    hidden_dim: int
    intermediate_dim: int
    dtype: int = ffi.DT_F32
    norm_eps: float = 1e-6


def dense_gated_mlp_graph(spec: DenseGatedMlpSpec, output_lifetime: int = ffi.LIFETIME_OUTPUT) -> ProgramGraph:
    """vyre_libs::nn::model::dense_gated_mlp_graph (dense_gated_mlp.rs:59-370) with the reference's own node programs,
    value names, shapes and lifetimes: learned RMSNorm of the residual stream (`mlp.norm`), bias-free gate / up projections
    (`linear_rows_no_bias_out_in_typed`), SwiGLU, bias-free down projection, residual add (`mlp.residual`). Weights are
    `Constant` values ([out, in] projections, [hidden] norm weight); the input is `residual`, the output `mlp.block_output`."""
    if min(spec.batch, spec.sequence, spec.hidden_dim, spec.intermediate_dim) <= 0:
        raise BackendError(ffi.ERR_INVALID_PROGRAM,
                           "Fix: dense gated MLP primitive construction failed: batch, sequence, hidden_dim, and intermediate_dim must be nonzero")
    if spec.dtype not in (ffi.DT_F16, ffi.DT_BF16, ffi.DT_F32):
        raise BackendError(ffi.ERR_INVALID_PROGRAM, "Fix: dense gated MLP primitive construction failed: dtype must be F16, BF16, or F32")
    rows, h, i, dt = spec.batch * spec.sequence, spec.hidden_dim, spec.intermediate_dim, spec.dtype
    if rows >= 1 << 32 or rows * max(h, i) >= 1 << 32 or h * i >= 1 << 32:
        raise BackendError(ffi.ERR_INVALID_PROGRAM, "Fix: dense gated MLP primitive construction failed: element counts overflow u32")
    inv, const = ffi.LIFETIME_INVOCATION, ffi.LIFETIME_CONSTANT
    ro, rw = ffi.ACCESS_READ_ONLY, ffi.ACCESS_READ_WRITE
    hidden_shape, inter_shape = [spec.batch, spec.sequence, h], [spec.batch, spec.sequence, i]
    read_hidden, write_hidden = value_contract(dt, hidden_shape, inv, ro), value_contract(dt, hidden_shape, inv, rw)
    read_inter, write_inter = value_contract(dt, inter_shape, inv, ro), value_contract(dt, inter_shape, inv, rw)
    norm_w, up_w, down_w = value_contract(dt, [h], const), value_contract(dt, [i, h], const), value_contract(dt, [h, i], const)
    graph = ProgramGraph()
    residual = graph.add_external_value("residual", read_hidden)
    norm_wv = graph.add_external_value("post_attention_layernorm.weight", norm_w)
    gate_w = graph.add_external_value("mlp.gate_proj.weight", up_w)
    up_wv = graph.add_external_value("mlp.up_proj.weight", up_w)
    down_wv = graph.add_external_value("mlp.down_proj.weight", down_w)
    _, (x,) = graph.add_node("mlp.norm", learned_rms_norm("input", "weight", "output", rows, h, spec.norm_eps, dt),
                             [("input", residual, read_hidden), ("weight", norm_wv, norm_w)], [("output", "mlp.normalized", write_hidden)])
    _, (gate,) = graph.add_node("mlp.gate_proj", linear_rows_no_bias_out_in_typed("input", "weight", "output", rows, h, i, dt),
                                [("input", x, read_hidden), ("weight", gate_w, up_w)], [("output", "mlp.gate", write_inter)])
    _, (up,) = graph.add_node("mlp.up_proj", linear_rows_no_bias_out_in_typed("input", "weight", "output", rows, h, i, dt),
                              [("input", x, read_hidden), ("weight", up_wv, up_w)], [("output", "mlp.up", write_inter)])
    _, (act,) = graph.add_node("mlp.swiglu", swiglu_typed("gate", "up", "output", rows * i, dt),
                               [("gate", gate, read_inter), ("up", up, read_inter)], [("output", "mlp.activated", write_inter)])
    _, (down,) = graph.add_node("mlp.down_proj", linear_rows_no_bias_out_in_typed("input", "weight", "output", rows, i, h, dt),
                                [("input", act, read_inter), ("weight", down_wv, down_w)], [("output", "mlp.down", write_hidden)])
    graph.add_node("mlp.residual", residual_add_typed("residual", "branch", "output", rows * h, dt),
                   [("residual", residual, read_hidden), ("branch", down, read_hidden)],
                   [("output", "mlp.block_output", value_contract(dt, hidden_shape, output_lifetime, rw))])
    return graph


# ---- scratch-reusing callers of the packed-int4 primitives (vyre-self-substrate/src/math/quantized_dispatch.rs) -----------
class QuantizedScratch:
    """Caller-owned scratch of the `*_via_with_scratch_into` wrappers: per (wrapper, shape) the compiled chain down to the
    ArtifactInstance, so that a repeated shape costs one submission. The reference keeps one scratch struct per wrapper
    (quantized_dispatch.rs:30-72); here one object serves all six. The dispatcher is the device it was made for."""

    def __init__(self, device: Device | None):
        out = C.c_void_p()
        check(ffi.lib().vyb_quantized_scratch_new(device._h if device is not None else None, C.byref(out)))
        self._h, self._dev = out, device

    def close(self) -> None:
        if self._h is not None:
            h, self._h = self._h, None
            ffi.lib().vyb_quantized_scratch_free(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def stats(self) -> dict:
        c, h, m = C.c_uint64(), C.c_uint64(), C.c_uint64()
        ffi.lib().vyb_quantized_scratch_stats(self._h, C.byref(c), C.byref(h), C.byref(m))
        return {"cached": c.value, "hits": h.value, "misses": m.value}


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def unpack_i4x8_via(scratch: QuantizedScratch, packed_words, lane_count: int) -> np.ndarray:
    """unpack.rs:14-84."""
    p, out = _u32(packed_words), np.empty(max(lane_count, 1), dtype=np.int32)
    check(ffi.lib().vyb_unpack_i4x8_via(scratch._h, p.ctypes.data, p.size, lane_count, out.ctypes.data))
    return out[:lane_count]


def i4x8_dot_f32_scaled_via(scratch: QuantizedScratch, lhs_packed, rhs_packed, lhs_scale: float, rhs_scale: float,
                            lane_count: int) -> float:
    """dot.rs:14-91."""
    a, b, out = _u32(lhs_packed), _u32(rhs_packed), np.empty(1, dtype=np.float32)
    check(ffi.lib().vyb_i4x8_dot_f32_scaled_via(scratch._h, a.ctypes.data, a.size, b.ctypes.data, b.size, lhs_scale, rhs_scale,
                                                lane_count, out.ctypes.data))
    return float(out[0])


def i4x8_matvec_f32_scaled_via(scratch: QuantizedScratch, weights_packed, x, row_scales, rows: int, cols: int) -> np.ndarray:
    """matvec.rs:14-110."""
    w, xv, rs, out = _u32(weights_packed), _f32(x), _f32(row_scales), np.empty(max(rows, 1), dtype=np.float32)
    check(ffi.lib().vyb_i4x8_matvec_f32_scaled_via(scratch._h, w.ctypes.data, w.size, xv.ctypes.data, xv.size, rs.ctypes.data,
                                                   rs.size, rows, cols, out.ctypes.data))
    return out[:rows]


def i4x8_batched_matvec_f32_scaled_via(scratch: QuantizedScratch, weights_packed, x_batches, row_scales, batch: int, rows: int,
                                       cols: int) -> np.ndarray:
    """batched_matvec.rs:14-132."""
    w, xv, rs = _u32(weights_packed), _f32(x_batches), _f32(row_scales)
    out = np.empty(max(batch * rows, 1), dtype=np.float32)
    check(ffi.lib().vyb_i4x8_batched_matvec_f32_scaled_via(scratch._h, w.ctypes.data, w.size, xv.ctypes.data, xv.size,
                                                           rs.ctypes.data, rs.size, batch, rows, cols, out.ctypes.data))
    return out[:batch * rows]


def i4x8_batched_matmul_f32_scaled_via(scratch: QuantizedScratch, weights_packed, activation_batches_packed, row_scales,
                                       batch_scales, batch: int, rows: int, cols: int) -> np.ndarray:
    """batched_matmul.rs:14-108."""
    w, a, rs, bs = _u32(weights_packed), _u32(activation_batches_packed), _f32(row_scales), _f32(batch_scales)
    out = np.empty(max(batch * rows, 1), dtype=np.float32)
    check(ffi.lib().vyb_i4x8_batched_matmul_f32_scaled_via(scratch._h, w.ctypes.data, w.size, a.ctypes.data, a.size,
                                                           rs.ctypes.data, rs.size, bs.ctypes.data, bs.size, batch, rows, cols,
                                                           out.ctypes.data))
    return out[:batch * rows]


def i4x8_batched_matmul_top1_f32_scaled_via(scratch: QuantizedScratch, weights_packed, activation_batches_packed, row_scales,
                                            batch_scales, batch: int, rows: int, cols: int):
    """top1.rs:14-126: (scores, indices)."""
    w, a, rs, bs = _u32(weights_packed), _u32(activation_batches_packed), _f32(row_scales), _f32(batch_scales)
    scores, idx = np.empty(max(batch, 1), dtype=np.float32), np.empty(max(batch, 1), dtype=np.uint32)
    check(ffi.lib().vyb_i4x8_batched_matmul_top1_f32_scaled_via(scratch._h, w.ctypes.data, w.size, a.ctypes.data, a.size,
                                                                rs.ctypes.data, rs.size, bs.ctypes.data, bs.size, batch, rows,
                                                                cols, scores.ctypes.data, idx.ctypes.data))
    return scores[:batch], idx[:batch]


# ---- the reference's wire frames (vyre-megakernel/src/lib.rs:1326-1355, envelope.rs:763-860) ---------------------------------
FRAME_VMK0, FRAME_VTP0, FRAME_VME0 = 0, 1, 2


def _take_frame(ptr, n) -> bytes:
    try:
        return C.string_at(ptr, n.value)
    finally:
        ffi.lib().vyb_frame_free(ptr)


def frame_encode(layer: int, body: bytes) -> bytes:
    out, n = C.c_void_p(), C.c_size_t()
    check(ffi.lib().vyb_frame_encode(layer, body, len(body), C.byref(out), C.byref(n)))
    return _take_frame(out, n)


def frame_decode(layer: int, frame: bytes) -> tuple[bytes, bytes]:
    """(body, digest) of an authenticated frame."""
    body, n, digest = C.c_void_p(), C.c_size_t(), C.create_string_buffer(32)
    buf = C.create_string_buffer(frame, len(frame))
    check(ffi.lib().vyb_frame_decode(layer, buf, len(frame), C.byref(body), C.byref(n), digest))
    return C.string_at(body, n.value), digest.raw


def payload_to_vtp0(payload: TargetPayload, neutral_artifact: bytes, node_id: int = 0, value_ids: list[int] | None = None) -> bytes:
    """TargetPayload::to_bytes of the reference for this backend's payload, bound to `neutral_artifact` (32 bytes)."""
    ids = (C.c_uint32 * max(1, len(value_ids or [])))(*(value_ids or []))
    out, n = C.c_void_p(), C.c_size_t()
    check(ffi.lib().vyb_payload_to_vtp0(payload._h, neutral_artifact, node_id, ids if value_ids else None, len(value_ids or []),
                                        C.byref(out), C.byref(n)))
    return _take_frame(out, n)


def payload_from_vtp0(frame: bytes) -> tuple[TargetPayload, bytes]:
    out, neutral = C.c_void_p(), C.create_string_buffer(32)
    check(ffi.lib().vyb_payload_from_vtp0(frame, len(frame), C.byref(out), neutral))
    return TargetPayload(out.value), neutral.raw


def envelope_to_vme0(vmk0: bytes, payload_frames: list[bytes]) -> bytes:
    k = len(payload_frames)
    ptrs = (C.c_char_p * max(1, k))(*payload_frames)
    lens = (C.c_size_t * max(1, k))(*[len(f) for f in payload_frames])
    out, n = C.c_void_p(), C.c_size_t()
    check(ffi.lib().vyb_envelope_to_vme0(vmk0, len(vmk0), ptrs, lens, k, C.byref(out), C.byref(n)))
    return _take_frame(out, n)


def envelope_from_vme0(frame: bytes) -> tuple[bytes, list[bytes]]:
    """(neutral artifact frame, payload frames) of an authenticated envelope."""
    count = C.c_uint32()
    check(ffi.lib().vyb_envelope_from_vme0(frame, len(frame), 0, None, None, C.byref(count)))
    parts = []
    for i in range(count.value + 1):
        out, n = C.c_void_p(), C.c_size_t()
        check(ffi.lib().vyb_envelope_from_vme0(frame, len(frame), i, C.byref(out), C.byref(n), None))
        parts.append(_take_frame(out, n))
    return parts[0], parts[1:]
