// Device, resident buffers, materialisation and submission: the ArtifactMaterializer / ArtifactInstance /
// Submission side of the contract (vyre-driver/src/backend/artifact_lifecycle.rs:100-186), implemented on the
// CUDA runtime. One library-owned non-blocking stream per instance (the reference forbids the legacy default
// stream, vyre-driver-cuda/src/backend/launch.rs:81-87). No CPU fallback anywhere: a missing device, a foreign
// handle or a wrong byte length is a structured error with "Fix:" text.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <unordered_map>

#include "../kernels/kernels.h"
#include "blake3.hpp"
#include "model.hpp"

using namespace vyb;

namespace {

std::atomic<uint64_t> g_next_owner{1};  // vyre-driver/src/backend/resource.rs:13 (starts at 1, never reused)

struct Resident {
    void* ptr = nullptr;
    size_t len = 0;
    uint32_t inflight = 0;
};

std::string cuda_msg(cudaError_t e) { return std::string(cudaGetErrorName(e)) + ": " + cudaGetErrorString(e); }

}  // namespace

struct vyb_device {
    // The handle given to the caller owns one reference; every instance materialised on the device owns
    // another, so an instance (or a completion) released after vyb_device_release never touches freed state.
    std::atomic<int> refs{1};
    int ordinal = 0;
    cudaDeviceProp prop{};
    uint64_t owner = 0;
    std::atomic<uint64_t> generation{1};
    std::atomic<bool> lost{false};
    std::string lost_reason;
    std::string device_name;
    std::mutex mu;
    std::unordered_map<uint64_t, Resident> residents;
    uint64_t next_id = 1;
    uint64_t resident_bytes = 0;

    int32_t check_alive(const char* what) {
        if (lost.load())
            return fail_device_lost(device_name, generation.load(), std::string(what) + " refused: " + lost_reason);
        return VYB_OK;
    }
    // vyre-driver/src/backend/resource.rs:61-84 (ResidentOwner::resolve) + resident.rs:196-201,426-434
    int32_t resolve(vyb_resident_handle h, const char* context, Resident** out) {
        if (h.owner != owner)
            return fail_invalid_program(
                std::string("Fix: ") + context + " received resident handle " + std::to_string(h.id) +
                " owned by backend instance " + std::to_string(h.owner) + ", but this instance is " +
                std::to_string(owner) +
                ". A resident handle is only valid on the backend instance that allocated it; reallocate and "
                "re-upload the buffer on this instance, or keep the original instance alive for as long as the "
                "handle is held.");
        auto it = residents.find(h.id);
        if (it == residents.end())
            return fail_invalid_program(std::string("Fix: ") + context + " received unknown or already freed resident handle " +
                                        std::to_string(h.id) + "; allocate it with vyb_alloc on this device first.");
        *out = &it->second;
        return VYB_OK;
    }
};

namespace {

struct PinnedBuf {
    void* ptr = nullptr;
    size_t cap = 0;
    bool in_use = false;
};
struct DeviceBuf {
    void* ptr = nullptr;
    size_t cap = 0;
    bool in_use = false;
};

}  // namespace

struct vyb_instance {
    std::atomic<int> refs{1};  // the caller's handle + one per live submission / completion
    vyb_device* dev = nullptr;
    Program program;
    uint32_t variant = 0;
    Digest artifact{}, payload{};
    vyb_device_identity identity{};
    uint64_t generation = 0;
    cudaStream_t stream = nullptr;
    std::mutex mu;
    std::vector<PinnedBuf> pinned;
    std::vector<DeviceBuf> temps;
    void* scratch = nullptr;  // op-specific device scratch, sized at materialisation
    size_t scratch_len = 0;
    uint32_t* status_dev = nullptr;   // 4 words, raised by kernels whose bounded waits ran out
    uint32_t* status_host = nullptr;  // pinned mirror

    // events are recycled: creating and destroying three per submission costs more than the launch itself
    std::vector<cudaEvent_t> timing_events, plain_events;
    cudaEvent_t acquire_event(bool timing) {
        auto& pool = timing ? timing_events : plain_events;
        if (!pool.empty()) {
            cudaEvent_t e = pool.back();
            pool.pop_back();
            return e;
        }
        cudaEvent_t e = nullptr;
        if (timing)
            cudaEventCreate(&e);
        else
            cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
        return e;
    }
    void release_event(cudaEvent_t e, bool timing) {
        if (e) (timing ? timing_events : plain_events).push_back(e);
    }

    void* acquire_pinned(size_t len) {
        for (auto& b : pinned)
            if (!b.in_use && b.cap >= len) {
                b.in_use = true;
                return b.ptr;
            }
        PinnedBuf b;
        if (cudaHostAlloc(&b.ptr, std::max<size_t>(len, 256), cudaHostAllocDefault) != cudaSuccess) return nullptr;
        b.cap = std::max<size_t>(len, 256);
        b.in_use = true;
        pinned.push_back(b);
        return b.ptr;
    }
    void release_pinned(void* p) {
        for (auto& b : pinned)
            if (b.ptr == p) b.in_use = false;
    }
    void* acquire_temp(size_t len) {
        for (auto& b : temps)
            if (!b.in_use && b.cap >= len) {
                b.in_use = true;
                return b.ptr;
            }
        DeviceBuf b;
        if (cudaMalloc(&b.ptr, std::max<size_t>(len, 256)) != cudaSuccess) return nullptr;
        b.cap = std::max<size_t>(len, 256);
        b.in_use = true;
        temps.push_back(b);
        return b.ptr;
    }
    void release_temp(void* p) {
        for (auto& b : temps)
            if (b.ptr == p) b.in_use = false;
    }
};

namespace {
void device_unref(vyb_device* d) {
    if (d && d->refs.fetch_sub(1) == 1) {
        cudaSetDevice(d->ordinal);
        for (auto& kv : d->residents) cudaFree(kv.second.ptr);
        delete d;
    }
}
void instance_unref(vyb_instance* i) {
    if (!i || i->refs.fetch_sub(1) != 1) return;
    cudaSetDevice(i->dev->ordinal);
    if (i->stream) {
        cudaStreamSynchronize(i->stream);
        cudaStreamDestroy(i->stream);
    }
    for (cudaEvent_t e : i->timing_events) cudaEventDestroy(e);
    for (cudaEvent_t e : i->plain_events) cudaEventDestroy(e);
    for (auto& b : i->pinned) cudaFreeHost(b.ptr);
    for (auto& b : i->temps) cudaFree(b.ptr);
    if (i->scratch) cudaFree(i->scratch);
    if (i->status_dev) cudaFree(i->status_dev);
    if (i->status_host) cudaFreeHost(i->status_host);
    device_unref(i->dev);
    delete i;
}

struct OutputSlot {
    uint32_t value_id = 0;
    void* dev_ptr = nullptr;
    size_t len = 0;
    void* host = nullptr;  // pinned readback target, nullptr when left resident
    bool direct = false;   // prepared sets: the kernel writes straight into `host` (mapped pinned memory), no copy node
};
}  // namespace

struct vyb_prepared;

struct vyb_submission {
    vyb_instance* inst = nullptr;
    cudaEvent_t start = nullptr, end = nullptr, done = nullptr;
    std::vector<void*> temps;
    std::vector<void*> staged;  // pinned copies of the caller's host inputs (the BindingSet owns its bytes)
    std::vector<OutputSlot> outputs;
    std::vector<uint64_t> resident_ids;
    uint32_t* status_host = nullptr;  // this submission's own pinned copy of the kernel status words
    vyb_prepared* prepared = nullptr;  // set when the submission replays a prepared graph (buffers belong to it)
    bool consumed = false;
};

// A validated binding set frozen into one CUDA graph: H2D of the host inputs, the kernels, D2H of the outputs and of
// the status words. Replayed with a single graph launch per submission.
struct vyb_prepared {
    vyb_instance* inst = nullptr;
    cudaGraphExec_t exec = nullptr;
    struct HostInput {
        uint32_t value_id;
        void* staging;  // pinned
        size_t len;
    };
    std::vector<HostInput> inputs;
    std::vector<OutputSlot> outputs;
    std::vector<void*> temps;
    std::vector<uint64_t> resident_ids;
    uint32_t* status_host = nullptr;
    cudaEvent_t done = nullptr;
    bool busy = false;  // one submission of a prepared set in flight at a time
};

struct vyb_completion {
    vyb_prepared* prepared = nullptr;  // outputs live in the prepared set's buffers; freeing the completion releases it
    vyb_instance* inst = nullptr;
    Digest artifact{};
    std::vector<OutputSlot> outputs;
    uint64_t device_ns = 0;
    bool has_device_ns = false;
};

namespace {

uint32_t rt_dtype(uint32_t tag) { return tag == VYB_DT_BF16 ? 1u : tag == VYB_DT_F16 ? 2u : 0u; }

// Programs whose kernels write every byte of every output: the zero fill of a backend-allocated output would be
// overwritten at once (the reference zero-fills because its generated kernels may skip padded elements).
bool overwrites_every_output_byte(const Program& p) {
    switch (p.kind) {
        case OpKind::LinearInt4GroupedRowmajor:
        case OpKind::LinearInt4Block:
        case OpKind::LinearInt8WeightOnly:
        case OpKind::LinearInt8Dynamic:
            return true;
        default:
            return false;
    }
}

// The int4 group-quantized projection y[batch][n] = x[batch][k] W^T by the kernel the payload names
cudaError_t run_int4_linear(vyb_instance* inst, uint32_t variant, const void* x, const void* w, const void* scale, void* y,
                            uint32_t batch, uint32_t k, uint32_t n, uint32_t group, uint32_t out_f32, cudaStream_t s) {
    using namespace vybk;
    const size_t out_elem = out_f32 ? 4 : 2;
    if (variant == KV_INT4_PREFILL_TCGEN05 && int4_prefill_supported(batch, n, k, group))
        return launch_int4_prefill(x, w, scale, y, batch, n, k, group, out_f32, inst->dev->prop.multiProcessorCount, s,
                                   inst->status_dev);
    if (variant == KV_INT4_GEMV_TMA && int4_gemv_supported(std::min(batch, 8u), n, k, group)) {
        for (uint32_t b0 = 0; b0 < batch; b0 += 8) {
            const uint32_t mb = std::min(8u, batch - b0);
            cudaError_t e = launch_int4_gemv((const uint16_t*)x + size_t(b0) * k, w, scale, (uint8_t*)y + size_t(b0) * n * out_elem,
                                             mb, n, k, out_f32, inst->dev->prop.multiProcessorCount, s, inst->status_dev);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    return launch_int4_linear_generic(x, w, scale, y, batch, n, k, group, out_f32, s);
}

// Launch the kernels of one program. `b[slot]` is the device pointer bound to the BufferDecl binding slot.
cudaError_t dispatch(vyb_instance* inst, void* const* b, cudaStream_t s) {
    const Program& p = inst->program;
    const uint32_t* u = p.params.u;
    using namespace vybk;
    switch (p.kind) {
        case OpKind::Linear4Bit:
            return launch_linear_4bit((const float*)b[0], (const uint32_t*)b[1], (const float*)b[2], (float*)b[3], u[0], u[1], s);
        case OpKind::Linear4BitAffineGrouped:
            if (inst->variant == KV_AFFINE_GROUPED_OUTPUT_MAJOR && affine_grouped_fast_supported(u[0], u[1], u[2], u[3]))
                return launch_affine_grouped_fast((const float*)b[0], (const uint32_t*)b[1], (const float*)b[2],
                                                  (const uint32_t*)b[3], (const float*)b[4], (float*)b[5], u[0], u[1], u[2],
                                                  u[3], inst->dev->prop.multiProcessorCount, s);
            return launch_linear_4bit_affine_grouped((const float*)b[0], (const uint32_t*)b[1], (const float*)b[2],
                                                     (const uint32_t*)b[3], (const float*)b[4], (float*)b[5], u[0], u[1],
                                                     u[2], u[3], s);
        case OpKind::I4Unpack: return launch_i4_unpack((const uint32_t*)b[0], (int32_t*)b[1], u[0], s);
        case OpKind::I4DotI32: return launch_i4_dot_i32((const uint32_t*)b[0], (const uint32_t*)b[1], (int32_t*)b[2], u[0], s);
        case OpKind::I4DotF32Scaled:
            return launch_i4_dot_f32_scaled((const uint32_t*)b[0], (const uint32_t*)b[1], (const float*)b[2],
                                            (const float*)b[3], (float*)b[4], u[0], s);
        case OpKind::I4BatchedMatvec:
            if (inst->variant == KV_I4_MATVEC_WARP_ROWS && i4_matvec_fast_supported(u[0], u[1], u[2]))
                return launch_i4_matvec_fast((const uint32_t*)b[0], (const float*)b[1], (const float*)b[2], (float*)b[3], u[0],
                                             u[1], u[2], s);
            return launch_i4_batched_matvec((const uint32_t*)b[0], (const float*)b[1], (const float*)b[2], (float*)b[3],
                                            u[0], u[1], u[2], s);
        case OpKind::I4BatchedMatmul:
            return launch_i4_batched_matmul((const uint32_t*)b[0], (const uint32_t*)b[1], (const float*)b[2],
                                            (const float*)b[3], (float*)b[4], u[0], u[1], u[2], s);
        case OpKind::I4BatchedMatmulTop1:
            return launch_i4_batched_matmul_top1((const uint32_t*)b[0], (const uint32_t*)b[1], (const float*)b[2],
                                                 (const float*)b[3], (float*)b[4], u[0], u[1], u[2], s);
        case OpKind::Int8Unpack:
            return launch_int8_unpack((const uint32_t*)b[0], (const float*)b[1], (float*)b[2], u[0], u[1], s);
        case OpKind::Int8Pack: return launch_int8_pack((const uint32_t*)b[0], (uint32_t*)b[1], u[0], s);
        case OpKind::LinearRows: {
            const bool has_bias = u[5] != 0;
            return launch_linear_rows(b[0], b[1], has_bias ? b[2] : nullptr, has_bias ? b[3] : b[2], u[0], u[1], u[2],
                                      rt_dtype(u[3]), u[4], s);
        }
        case OpKind::MatmulU32: {  // u[3]: bias bound at slot 2, output at slot 3
            const bool has_bias = u[3] != 0;
            return launch_matmul_u32((const uint32_t*)b[0], (const uint32_t*)b[1], has_bias ? (const uint32_t*)b[2] : nullptr,
                                     (uint32_t*)(has_bias ? b[3] : b[2]), u[0], u[1], u[2], s);
        }
        case OpKind::MoeGate: return launch_moe_gate((const float*)b[0], (uint32_t*)b[1], (float*)b[2], u[2], u[0], u[1], s);
        case OpKind::SoftmaxTopK:
            return launch_softmax_top_k((const float*)b[0], (uint32_t*)b[1], (float*)b[2], (float*)b[3], (uint32_t*)b[4],
                                        u[0], u[1], s);
        case OpKind::TopK:
            return launch_top_k((const float*)b[0], (uint32_t*)b[1], (float*)b[2], (uint32_t*)b[3], u[0], u[1], s);
        case OpKind::Swiglu: return launch_swiglu(b[0], b[1], b[2], u[0], rt_dtype(u[1]), s);
        case OpKind::ResidualAdd: return launch_residual_add(b[0], b[1], b[2], u[0], rt_dtype(u[1]), s);
        case OpKind::RmsNorm: {
            float eps;
            std::memcpy(&eps, &u[2], 4);
            const bool gated = u[5] != 0;
            return launch_rms_norm(b[0], b[1], gated ? b[2] : nullptr, gated ? b[3] : b[2], u[0], u[1], eps, rt_dtype(u[3]),
                                   rt_dtype(u[4]), inst->variant == KV_RMS_NORM_TREE, s);
        }
        case OpKind::KQuantUnpack:
            return launch_k_quant_unpack((const uint32_t*)b[0], (const float*)b[1], (const float*)b[2], (float*)b[3], u[0], u[1], s);
        case OpKind::KQuantLinear:
            if (inst->variant == KV_K_QUANT_WORD_COLUMNS && k_quant_linear_fast_supported(u[0], u[1], u[2]))
                return launch_k_quant_linear_fast((const float*)b[0], (const uint32_t*)b[1], (const float*)b[2], (const float*)b[3],
                                                  (const float*)b[4], (float*)b[5], (float*)inst->scratch, u[0], u[1], u[2],
                                                  inst->dev->prop.multiProcessorCount, s);
            return launch_k_quant_linear((const float*)b[0], (const uint32_t*)b[1], (const float*)b[2], (const float*)b[3],
                                         (const float*)b[4], (float*)b[5], u[0], u[1], u[2], s);
        case OpKind::ExpertMlp:
            return launch_expert_mlp((const float*)b[0], (const float*)b[1], (const float*)b[2], (const float*)b[3],
                                     (const float*)b[4], (const float*)b[5], (const float*)b[6], (float*)b[7],
                                     (float*)inst->scratch, u[0], u[1], u[2], s);
        case OpKind::MoeLayerAccumulate:
            return launch_moe_layer_accumulate((const float*)b[4], (const float*)b[5], (float*)b[6], u[3], u[2], s);
        case OpKind::LinearInt4GroupedRowmajor: {
            return run_int4_linear(inst, inst->variant, b[0], b[1], b[2], b[3], u[0], u[1], u[2], u[3],
                                   u[4] == VYB_DT_F32 ? 1u : 0u, s);
        }
        case OpKind::LinearInt4Block: {
            // slots: x, [norm weight], packed weights, scales, [gate | residual], out
            const uint32_t batch = u[0], k = u[1], n = u[2], group = u[3], parts = u[5];
            float eps;
            std::memcpy(&eps, &u[6], 4);
            uint32_t slot = 0;
            const void* x = b[slot++];
            const void* norm_w = (parts & 1u) ? b[slot++] : nullptr;
            const void* w = b[slot++];
            const void* scale = b[slot++];
            const void* gate = (parts & 4u) ? b[slot++] : nullptr;
            const void* resid = (parts & 2u) ? b[slot++] : nullptr;
            void* y = b[slot];
            const int sms = inst->dev->prop.multiProcessorCount;
            const bool gemv = inst->variant == KV_INT4_BLOCK_GEMV;
            // whole rows of 2048 / 4096, one or two batch rows: norm, projection and SwiGLU / residual add are ONE launch
            if (gemv && batch <= 2 && int4_gemv_halfsm_supported(batch, n, k, group))
                return launch_int4_gemv_halfsm(x, w, scale, y, batch, n, k, 0, sms, s, inst->status_dev, false, nullptr, 0, false,
                                               norm_w, eps, resid, gate);
            // otherwise the stand-alone kernels in sequence: the norm into scratch (the tree form from 2048 elements on, as
            // the stand-alone operator chooses), the projection, SwiGLU / the residual add in place
            if (norm_w) {
                cudaError_t e = launch_rms_norm(x, norm_w, nullptr, inst->scratch, batch, k, eps, 1, 1, k >= 2048, s);
                if (e != cudaSuccess) return e;
                x = inst->scratch;
            }
            if (gemv && int4_gemv_kblocks_supported(batch, n, k, group)) {
                // long rows: SwiGLU / the residual add where the last-arriving k block rounds the sums
                bool fused = false;
                cudaError_t e = launch_int4_gemv_kblocks(x, w, scale, y, batch, n, k, 0, sms, s, false, resid, gate, &fused);
                if (e != cudaSuccess || fused) return e;
            } else {
                cudaError_t e = run_int4_linear(inst, gemv ? uint32_t(KV_INT4_GEMV_TMA) : inst->variant, x, w, scale, y, batch, k, n,
                                                group, 0, s);
                if (e != cudaSuccess) return e;
            }
            if (gate) return launch_swiglu(gate, y, y, batch * n, 1, s);
            return resid ? launch_residual_add(resid, y, y, batch * n, 1, s) : cudaSuccess;
        }
        case OpKind::LinearInt8Dynamic: {
            const uint32_t rows = u[0], k = u[1], n = u[2];
            if (!int8_gemm_supported(rows, n, k)) return cudaErrorNotSupported;
            int8_t* xq = static_cast<int8_t*>(inst->scratch);  // [rows, k] quantised activations
            cudaError_t e = launch_quantize_per_token_int8(b[0], xq, (float*)b[2], rows, k, s);
            if (e != cudaSuccess) return e;
            return launch_int8_gemm(xq, (const int8_t*)b[1], (int32_t*)b[3], rows, n, k,
                                    inst->dev->prop.multiProcessorCount, s, inst->status_dev);
        }
        case OpKind::MoeFfnInt4: {
            const uint32_t tokens = u[0], hidden = u[1], inter = u[2], experts = u[3], topk = u[4], group = u[5];
            if (!moe_ffn_int4_supported(tokens, hidden, inter, experts, topk, group)) return cudaErrorNotSupported;
            return launch_moe_ffn_int4(b[0], b[1], b[2], b[3], b[4], b[5], b[6], (uint32_t*)b[7], (float*)b[8],
                                       inst->scratch, tokens, hidden, inter, experts, topk, group,
                                       inst->dev->prop.multiProcessorCount, s, inst->status_dev);
        }
        case OpKind::LinearInt8WeightOnly:
            return launch_int8_weight_only_linear((const float*)b[0], (const int8_t*)b[1], (const float*)b[2],
                                                  (float*)b[3], u[0], u[2], u[1], s);
        default: return cudaErrorNotSupported;
    }
}

size_t scratch_bytes_for(const Program& p) {
    switch (p.kind) {
        case OpKind::ExpertMlp: return size_t(p.params.u[1]) * 4;
        case OpKind::LinearInt8Dynamic: return size_t(p.params.u[0]) * p.params.u[1];
        case OpKind::KQuantLinear: return vybk::k_quant_linear_fast_scratch_bytes(p.params.u[1]);
        case OpKind::LinearInt4Block:  // the normalised activations, when the norm runs as its own kernel
            return (p.params.u[5] & 1u) ? size_t(p.params.u[0]) * p.params.u[1] * 2 : 0;
        case OpKind::MoeFfnInt4:
            return vybk::moe_ffn_int4_scratch_bytes(p.params.u[0], p.params.u[1], p.params.u[2], p.params.u[3], p.params.u[4]);
        default: return 0;
    }
}

// every op kind has a kernel; the fused MoE layer additionally needs shapes its grouped tensor-core GEMM accepts
bool program_supported(const Program& p, std::string* why) {
    if (p.kind == OpKind::MoeFfnInt4) {
        const uint32_t* u = p.params.u;
        if (!vybk::moe_ffn_int4_supported(u[0], u[1], u[2], u[3], u[4], u[5])) {
            *why = "operator `" + p.op_id + "` with hidden=" + std::to_string(u[1]) + " inter=" + std::to_string(u[2]) +
                   " experts=" + std::to_string(u[3]) + " topk=" + std::to_string(u[4]) + " group=" + std::to_string(u[5]) +
                   " (needs hidden and inter multiples of 256, group a multiple of 64, experts <= 64, topk <= 8)";
            return false;
        }
    }
    return true;
}

}  // namespace

extern "C" {

// ---- Device --------------------------------------------------------------------------------------------------
int32_t vyb_device_acquire(int32_t ordinal, vyb_device** device) {
    if (!device) return fail_invalid_program("Fix: pass a non-null device out-pointer.");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail_dispatch(int(e), "no CUDA device is visible to this process (" + cuda_msg(e) +
                                         "); the native backend has no CPU path");
    }
    if (ordinal < 0 || ordinal >= count)
        return fail_dispatch(int(cudaErrorInvalidDevice), "device ordinal " + std::to_string(ordinal) +
                                                              " is out of range for " + std::to_string(count) +
                                                              " visible device(s)");
    auto d = std::make_unique<vyb_device>();
    d->ordinal = ordinal;
    e = cudaGetDeviceProperties(&d->prop, ordinal);
    if (e != cudaSuccess) return fail_dispatch(int(e), "cudaGetDeviceProperties failed: " + cuda_msg(e));
    if (d->prop.major != 10)
        return fail_unsupported("sm_" + std::to_string(d->prop.major) + std::to_string(d->prop.minor) +
                                " device (the native kernels are built for sm_100a only)");
    e = cudaSetDevice(ordinal);
    if (e != cudaSuccess) return fail_dispatch(int(e), "cudaSetDevice failed: " + cuda_msg(e));
    d->owner = g_next_owner.fetch_add(1);
    d->device_name = "cuda:" + std::to_string(ordinal) + ":" + d->prop.name;
    *device = d.release();
    clear_error();
    return VYB_OK;
}

int32_t vyb_device_identity_of(const vyb_device* d, vyb_device_identity* out) {
    if (!d || !out) return fail_invalid_program("Fix: pass a non-null device and identity out-pointer.");
    std::snprintf(out->backend, sizeof(out->backend), "%s", BACKEND_ID);
    std::snprintf(out->device, sizeof(out->device), "%s", d->device_name.c_str());
    out->generation = d->generation.load();
    return VYB_OK;
}

int32_t vyb_device_caps_of(const vyb_device* d, vyb_device_caps* out) {
    if (!d || !out) return fail_invalid_program("Fix: pass a non-null device and caps out-pointer.");
    *out = vyb_device_caps{};
    std::snprintf(out->name, sizeof(out->name), "%s", d->prop.name);
    out->ordinal = d->ordinal;
    out->compute_major = d->prop.major;
    out->compute_minor = d->prop.minor;
    out->total_memory = d->prop.totalGlobalMem;
    out->max_threads_per_block = d->prop.maxThreadsPerBlock;
    out->shared_memory_per_block = int32_t(d->prop.sharedMemPerBlock);
    out->shared_memory_per_sm = int32_t(d->prop.sharedMemPerMultiprocessor);
    out->shared_memory_per_block_optin = int32_t(d->prop.sharedMemPerBlockOptin);
    out->warp_size = d->prop.warpSize;
    out->cooperative_launch = d->prop.cooperativeLaunch;
    out->multi_processor_count = d->prop.multiProcessorCount;
    out->l2_cache_bytes = d->prop.l2CacheSize;
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, d->ordinal) == cudaSuccess) out->memory_clock_rate_khz = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, d->ordinal) == cudaSuccess) out->core_clock_rate_khz = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, d->ordinal) == cudaSuccess)
        out->global_memory_bus_width_bits = v;
    return VYB_OK;
}

int32_t vyb_device_is_healthy(const vyb_device* d) { return d && !d->lost.load() ? 1 : 0; }

int32_t vyb_device_mark_lost(vyb_device* d, const char* reason) {
    if (!d) return fail_invalid_program("Fix: pass a non-null device.");
    std::lock_guard<std::mutex> lk(d->mu);
    d->lost_reason = reason ? reason : "device marked lost by the host";
    d->lost.store(true);
    return VYB_OK;
}

int32_t vyb_device_reacquire(vyb_device* d) {
    if (!d) return fail_invalid_program("Fix: pass a non-null device.");
    std::lock_guard<std::mutex> lk(d->mu);
    // handles of the lost generation are stale: drop the table (memory of a really lost context is gone;
    // for the host-injected case the buffers are released here)
    for (auto& kv : d->residents) cudaFree(kv.second.ptr);
    d->residents.clear();
    d->resident_bytes = 0;
    d->owner = g_next_owner.fetch_add(1);
    d->generation.fetch_add(1);
    d->lost.store(false);
    d->lost_reason.clear();
    return VYB_OK;
}

void vyb_device_release(vyb_device* d) { device_unref(d); }
void vyb_device_retain(vyb_device* d) {
    if (d) d->refs.fetch_add(1);
}

// ---- resident buffers (vyre-driver-cuda/src/backend/resident.rs) -------------------------------------------------
int32_t vyb_alloc(vyb_device* d, size_t byte_len, vyb_resident_handle* out) {
    if (!d || !out) return fail_invalid_program("Fix: pass a non-null device and handle out-pointer.");
    if (int32_t rc = d->check_alive("resident allocation")) return rc;
    if (byte_len == 0)
        return fail_invalid_program(
            "Fix: resident allocation of 0 bytes is refused; allocate at least one byte or skip the buffer.");
    cudaSetDevice(d->ordinal);
    size_t free_b = 0, total_b = 0;
    cudaMemGetInfo(&free_b, &total_b);
    if (byte_len > free_b) return fail_oom(byte_len, free_b);
    void* ptr = nullptr;
    cudaError_t e = cudaMalloc(&ptr, byte_len);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_oom(byte_len, free_b);
    }
    std::lock_guard<std::mutex> lk(d->mu);
    uint64_t id = d->next_id++;
    d->residents[id] = Resident{ptr, byte_len, 0};
    d->resident_bytes += byte_len;
    out->owner = d->owner;
    out->id = id;
    clear_error();
    return VYB_OK;
}

int32_t vyb_upload_at(vyb_device* d, vyb_resident_handle h, size_t offset_bytes, const void* bytes, size_t len) {
    if (!d || (!bytes && len)) return fail_invalid_program("Fix: pass a non-null device and source bytes.");
    if (int32_t rc = d->check_alive("resident upload")) return rc;
    void* dst;
    {
        std::lock_guard<std::mutex> lk(d->mu);
        Resident* r = nullptr;
        if (int32_t rc = d->resolve(h, "CUDA resident upload", &r)) return rc;
        if (offset_bytes > r->len || len > r->len - offset_bytes)
            return fail_invalid_program("Fix: resident upload of " + std::to_string(len) + " bytes at offset " +
                                        std::to_string(offset_bytes) + " exceeds the " + std::to_string(r->len) +
                                        "-byte allocation; allocate a larger buffer or split the upload.");
        // a dispatch in flight may be reading or writing the buffer on another stream (resident.rs:185-190, 287-364)
        if (r->inflight)
            return fail_invalid_program("Fix: resident buffer is bound to a dispatch in flight; wait for the pending "
                                        "submission (or free the prepared set that holds it) before uploading.");
        r->inflight++;  // keeps vyb_free away while the copy runs
        dst = static_cast<uint8_t*>(r->ptr) + offset_bytes;
    }
    cudaSetDevice(d->ordinal);
    cudaError_t e = cudaMemcpy(dst, bytes, len, cudaMemcpyHostToDevice);
    // a copy from pageable memory may return once the bytes are staged, before the DMA has landed; submissions run on
    // non-blocking streams that do not order themselves behind it, so the upload ends only when the copy has
    if (e == cudaSuccess) e = cudaStreamSynchronize(cudaStreamLegacy);
    {
        std::lock_guard<std::mutex> lk(d->mu);
        auto it = d->residents.find(h.id);
        if (it != d->residents.end() && it->second.inflight) it->second.inflight--;
    }
    if (e != cudaSuccess) return fail_dispatch(int(e), "resident upload failed: " + cuda_msg(e));
    clear_error();
    return VYB_OK;
}
int32_t vyb_upload(vyb_device* d, vyb_resident_handle h, const void* bytes, size_t len) {
    return vyb_upload_at(d, h, 0, bytes, len);
}

int32_t vyb_download_range(vyb_device* d, vyb_resident_handle h, size_t offset_bytes, void* dst, size_t len) {
    if (!d || (!dst && len)) return fail_invalid_program("Fix: pass a non-null device and destination.");
    if (int32_t rc = d->check_alive("resident download")) return rc;
    const void* src;
    {
        std::lock_guard<std::mutex> lk(d->mu);
        Resident* r = nullptr;
        if (int32_t rc = d->resolve(h, "CUDA resident download", &r)) return rc;
        if (offset_bytes > r->len || len > r->len - offset_bytes)
            return fail_invalid_program("Fix: resident download of " + std::to_string(len) + " bytes at offset " +
                                        std::to_string(offset_bytes) + " exceeds the " + std::to_string(r->len) +
                                        "-byte allocation.");
        r->inflight++;  // keeps vyb_free away while the copy runs; reading beside a dispatch in flight is the caller's call
        src = static_cast<const uint8_t*>(r->ptr) + offset_bytes;
    }
    cudaSetDevice(d->ordinal);
    cudaError_t e = cudaMemcpy(dst, src, len, cudaMemcpyDeviceToHost);
    {
        std::lock_guard<std::mutex> lk(d->mu);
        auto it = d->residents.find(h.id);
        if (it != d->residents.end() && it->second.inflight) it->second.inflight--;
    }
    if (e != cudaSuccess) return fail_dispatch(int(e), "resident download failed: " + cuda_msg(e));
    clear_error();
    return VYB_OK;
}
int32_t vyb_download(vyb_device* d, vyb_resident_handle h, void* dst, size_t len) {
    return vyb_download_range(d, h, 0, dst, len);
}

int32_t vyb_free(vyb_device* d, vyb_resident_handle h) {
    if (!d) return fail_invalid_program("Fix: pass a non-null device.");
    std::lock_guard<std::mutex> lk(d->mu);
    Resident* r = nullptr;
    if (int32_t rc = d->resolve(h, "CUDA resident free", &r)) return rc;
    if (r->inflight != 0)
        return fail_invalid_program("Fix: resident handle " + std::to_string(h.id) +
                                    " is still bound to an in-flight dispatch; wait for the submission before freeing it.");
    cudaFree(r->ptr);
    d->resident_bytes -= r->len;
    d->residents.erase(h.id);
    clear_error();
    return VYB_OK;
}

int32_t vyb_resident_device_ptr(vyb_device* d, vyb_resident_handle h, void** device_ptr, size_t* len) {
    if (!d || !device_ptr) return fail_invalid_program("Fix: pass a non-null device and pointer out-pointer.");
    std::lock_guard<std::mutex> lk(d->mu);
    Resident* r = nullptr;
    if (int32_t rc = d->resolve(h, "CUDA resident pointer query", &r)) return rc;
    *device_ptr = r->ptr;
    if (len) *len = r->len;
    return VYB_OK;
}

// ---- materialise: vyre-driver/src/materialize.rs:81-146 (admit), fail closed ------------------------------------------
int32_t vyb_materialize(vyb_device* d, const vyb_artifact* artifact, const vyb_payload* payload,
                        vyb_instance** instance) {
    if (!d || !artifact || !payload || !instance)
        return fail_invalid_program("Fix: pass non-null device, artifact, payload and instance out-pointer.");
    if (int32_t rc = d->check_alive("materialisation")) return rc;
    const Payload& pl = payload->p;
    auto invalid_module = [](const std::string& m) {
        return fail_invalid_program("Fix: " + m + "; recompile the artifact with this backend's target compiler.");
    };
    if (pl.neutral_artifact != artifact->a.digest)
        return invalid_module("target payload is not authenticated for the supplied neutral artifact");
    if (pl.format != PAYLOAD_FORMAT || pl.format_version != PAYLOAD_FORMAT_VERSION)
        return fail_unsupported("target payload format `" + pl.format + "`");
    if (!profile_equal(pl.profile, native_profile()))
        return invalid_module("target payload profile does not match the acquired materializer profile");
    {
        // re-authenticate the bytes: a payload edited after sealing must not materialise
        Payload check;
        std::string err;
        if (!Payload::from_bytes(pl.bytes.data(), pl.bytes.size(), &check, &err) || check.digest != pl.digest)
            return invalid_module("target payload bytes fail authentication (" + err + ")");
    }
    if (pl.modules.size() != 1)
        return invalid_module("target module count must equal the compiler-selected fusion-group count");
    const TargetModule& m = pl.modules[0];
    if (m.entry_point != "main") return invalid_module("target module entry point must be `main`");
    Program prog;
    std::string err;
    if (!Program::from_wire(m.program_wire.data(), m.program_wire.size(), &prog, &err))
        return invalid_module("selected Program is malformed: " + err);
    if (prog.fingerprint() != artifact->a.program.fingerprint())
        return invalid_module("target module group/stage/node identity must match the neutral selected plan");
    if (prog.trap) return fail_invalid_program(prog.trap_message);
    if (m.kernel_variant != select_kernel_variant(prog))
        return invalid_module("target module kernel variant disagrees with the op spec");
    {
        std::string why;
        if (!program_supported(prog, &why)) return fail_unsupported(why);
    }

    cudaSetDevice(d->ordinal);
    auto inst = std::make_unique<vyb_instance>();
    inst->dev = d;
    inst->program = std::move(prog);
    inst->variant = m.kernel_variant;
    inst->artifact = artifact->a.digest;
    inst->payload = pl.digest;
    vyb_device_identity_of(d, &inst->identity);
    inst->generation = d->generation.load();
    cudaError_t e = cudaStreamCreateWithFlags(&inst->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return fail_dispatch(int(e), "stream creation failed: " + cuda_msg(e));
    inst->scratch_len = scratch_bytes_for(inst->program);
    if (inst->scratch_len) {
        e = cudaMalloc(&inst->scratch, inst->scratch_len);
        if (e != cudaSuccess) {
            cudaGetLastError();
            cudaStreamDestroy(inst->stream);
            return fail_oom(inst->scratch_len, 0);
        }
    }
    e = cudaMalloc(reinterpret_cast<void**>(&inst->status_dev), 16);
    if (e == cudaSuccess) e = cudaMemset(inst->status_dev, 0, 16);
    if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void**>(&inst->status_host), 16, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "status buffer allocation failed: " + cuda_msg(e));
    }
    std::memset(inst->status_host, 0, 16);
    d->refs.fetch_add(1);
    *instance = inst.release();
    clear_error();
    return VYB_OK;
}

void vyb_instance_artifact_digest(const vyb_instance* i, uint8_t out[32]) { std::memcpy(out, i->artifact.data(), 32); }
void vyb_instance_payload_digest(const vyb_instance* i, uint8_t out[32]) { std::memcpy(out, i->payload.data(), 32); }
int32_t vyb_instance_device(const vyb_instance* i, vyb_device_identity* out) {
    if (!i || !out) return fail_invalid_program("Fix: pass a non-null instance and identity out-pointer.");
    *out = i->identity;
    return VYB_OK;
}
void vyb_instance_free(vyb_instance* i) { instance_unref(i); }

// ---- submit (vyre-driver-cuda/src/materializer.rs:165-283) -------------------------------------------------------------
int32_t vyb_submit(vyb_instance* inst, const uint8_t artifact_digest[32], const vyb_binding* bindings,
                   size_t n_bindings, const vyb_dispatch_config* config, vyb_submission** submission) {
    if (!inst || !artifact_digest || !submission || (!bindings && n_bindings))
        return fail_invalid_program("Fix: pass non-null instance, artifact digest, bindings and submission out-pointer.");
    vyb_device* d = inst->dev;
    if (int32_t rc = d->check_alive("submission")) return rc;
    if (inst->generation != d->generation.load())
        return fail_device_lost(d->device_name, inst->generation,
                                "the instance belongs to a previous device generation");
    if (std::memcmp(artifact_digest, inst->artifact.data(), 32) != 0)
        return fail_invalid_program(
            "Fix: the binding set was built for a different artifact than this instance; rebuild the bindings from the "
            "session that owns the instance.");
    bool leave_resident = false;
    if (config) {
        const bool any_grid = config->grid_override[0] || config->grid_override[1] || config->grid_override[2];
        if (any_grid)
            for (int a = 0; a < 3; ++a)
                if (config->grid_override[a] == 0)
                    return fail_invalid_program("Fix: invocation grid axis " + std::to_string(a) +
                                                " must be positive, got 0.");
        if (config->workgroup_override[0] || config->workgroup_override[1] || config->workgroup_override[2])
            return fail_unsupported("DispatchConfig.workgroup_override (hand-written kernels fix their launch shape)");
        if (config->ulp_budget) return fail_unsupported("DispatchConfig.ulp_budget");
        if (config->max_output_bytes) return fail_unsupported("DispatchConfig.max_output_bytes");
        if (config->cooperative) return fail_unsupported("DispatchConfig.cooperative");
        leave_resident = config->leave_resident != 0;
    }
    const Program& p = inst->program;
    std::lock_guard<std::mutex> ilk(inst->mu);
    cudaSetDevice(d->ordinal);

    auto sub = std::make_unique<vyb_submission>();
    sub->inst = inst;
    void* slot_ptr[16] = {nullptr};
    auto cleanup = [&]() {
        for (void* t : sub->temps) inst->release_temp(t);
        for (void* t : sub->staged) inst->release_pinned(t);
        if (sub->status_host) inst->release_pinned(sub->status_host);
        for (auto& o : sub->outputs)
            if (o.host) inst->release_pinned(o.host);
        std::lock_guard<std::mutex> lk(d->mu);
        for (uint64_t id : sub->resident_ids) {
            auto it = d->residents.find(id);
            if (it != d->residents.end() && it->second.inflight) it->second.inflight--;
        }
    };
    for (size_t i = 0; i < n_bindings; ++i) {
        if (!p.buffer_by_binding(bindings[i].value_id)) {
            cleanup();
            return fail_invalid_program("Fix: binding names value id " + std::to_string(bindings[i].value_id) +
                                        ", which this artifact does not declare; bind only the program's buffer slots.");
        }
    }
    for (const BufferDecl& bd : p.buffers) {
        if (bd.access == VYB_ACCESS_WORKGROUP) continue;
        if (bd.binding >= 16) {
            cleanup();
            return fail_invalid_program("Fix: binding slot exceeds the 16 slots this backend supports.");
        }
        const size_t need = size_t(bd.count) * dtype_size_bytes(bd.dtype);
        const size_t logical = bd.has_output_byte_range ? size_t(bd.output_byte_end - bd.output_byte_begin) : need;
        const vyb_binding* b = nullptr;
        for (size_t i = 0; i < n_bindings; ++i)
            if (bindings[i].value_id == bd.binding) b = &bindings[i];
        const bool is_input = bd.access == VYB_ACCESS_READ_ONLY || bd.access == VYB_ACCESS_READ_WRITE;
        const bool is_output = bd.access == VYB_ACCESS_OUTPUT || bd.access == VYB_ACCESS_READ_WRITE;
        void* dev_ptr = nullptr;
        bool resident = false;
        if (b && b->kind == VYB_BIND_RESIDENT) {
            std::lock_guard<std::mutex> lk(d->mu);
            Resident* r = nullptr;
            if (int32_t rc = d->resolve(b->resident, "CUDA resident dispatch", &r)) {
                cleanup();
                return rc;
            }
            // an output may be bound with its logical (trimmed) size; inputs need the declared size
            const size_t min_len = bd.access == VYB_ACCESS_OUTPUT ? logical : need;
            if (r->len < min_len) {
                cleanup();
                return fail_invalid_program("Fix: resident buffer bound to `" + bd.name + "` holds " +
                                            std::to_string(r->len) + " bytes but the program needs " +
                                            std::to_string(min_len) + "; allocate the declared size.");
            }
            r->inflight++;
            sub->resident_ids.push_back(b->resident.id);
            dev_ptr = r->ptr;
            resident = true;
        } else if (b && b->kind == VYB_BIND_HOST) {
            const bool placeholder_ok = bd.access == VYB_ACCESS_OUTPUT && (b->len == logical || b->len == need);
            if (b->len != need && !placeholder_ok) {
                cleanup();
                return fail_invalid_program("Fix: host bytes bound to `" + bd.name + "` are " + std::to_string(b->len) +
                                            " bytes but the program declares " + std::to_string(need) +
                                            "; bind exactly count * element size bytes.");
            }
            if (!b->host_ptr && b->len) {
                cleanup();
                return fail_invalid_program("Fix: host binding for `" + bd.name + "` has a null pointer.");
            }
        } else if (b) {
            cleanup();
            return fail_invalid_program("Fix: binding kind must be VYB_BIND_HOST or VYB_BIND_RESIDENT.");
        } else if (bd.access != VYB_ACCESS_OUTPUT) {
            cleanup();
            return fail_invalid_program("Fix: missing input for buffer `" + bd.name + "` (slot " +
                                        std::to_string(bd.binding) + "); bind every ReadOnly and ReadWrite buffer.");
        }
        if (!resident) {
            dev_ptr = inst->acquire_temp(need);
            if (!dev_ptr) {
                cleanup();
                return fail_oom(need, 0);
            }
            sub->temps.push_back(dev_ptr);
            cudaError_t e = cudaSuccess;
            if (is_input) {
                // host bytes are copied in at submit, as BindingSet::insert_host does
                // (vyre-driver/src/backend/artifact_lifecycle.rs:34-96): the caller may reuse its buffer at once
                void* stage = inst->acquire_pinned(need);
                if (!stage) {
                    cleanup();
                    return fail_oom(need, 0);
                }
                sub->staged.push_back(stage);
                std::memcpy(stage, b->host_ptr, need);
                e = cudaMemcpyAsync(dev_ptr, stage, need, cudaMemcpyHostToDevice, inst->stream);
            } else if (!overwrites_every_output_byte(p)) {
                e = cudaMemsetAsync(dev_ptr, 0, need, inst->stream);  // backend-allocated outputs start zeroed
            }
            if (e != cudaSuccess) {
                cleanup();
                return fail_dispatch(int(e), "input staging failed: " + cuda_msg(e));
            }
        }
        slot_ptr[bd.binding] = dev_ptr;
        if (is_output) {
            OutputSlot o;
            o.value_id = bd.binding;
            o.dev_ptr = static_cast<uint8_t*>(dev_ptr) + (bd.has_output_byte_range ? bd.output_byte_begin : 0);
            o.len = logical;
            if (!(resident && leave_resident)) {
                o.host = inst->acquire_pinned(logical);
                if (!o.host) {
                    cleanup();
                    return fail_oom(logical, 0);
                }
            }
            sub->outputs.push_back(o);
        }
    }
    sub->start = inst->acquire_event(true);  // inst->mu is held for the whole submission
    sub->end = inst->acquire_event(true);
    sub->done = inst->acquire_event(false);
    cudaEventRecord(sub->start, inst->stream);
    cudaGetLastError();  // a non-sticky error left by an unrelated earlier call must not be blamed on this launch
    cudaError_t e = dispatch(inst, slot_ptr, inst->stream);
    cudaEventRecord(sub->end, inst->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        cudaStreamSynchronize(inst->stream);
        cleanup();
        inst->release_event(sub->start, true);
        inst->release_event(sub->end, true);
        inst->release_event(sub->done, false);
        if (e == cudaErrorNotSupported) return fail_unsupported("operator `" + p.op_id + "`");
        return fail_dispatch(int(e), "kernel launch failed: " + cuda_msg(e));
    }
    for (auto& o : sub->outputs)
        if (o.host) cudaMemcpyAsync(o.host, o.dev_ptr, o.len, cudaMemcpyDeviceToHost, inst->stream);
    // every submission reads the status words into its OWN pinned slot and clears them on the stream right after,
    // so a word raised by one submission is never reported for another
    sub->status_host = static_cast<uint32_t*>(inst->acquire_pinned(16));
    if (sub->status_host) {
        sub->status_host[0] = 0;
        cudaMemcpyAsync(sub->status_host, inst->status_dev, 16, cudaMemcpyDeviceToHost, inst->stream);
        cudaMemsetAsync(inst->status_dev, 0, 16, inst->stream);
    }
    cudaEventRecord(sub->done, inst->stream);
    inst->refs.fetch_add(1);  // released by the completion (or by a failed wait)
    *submission = sub.release();
    clear_error();
    return VYB_OK;
}

int32_t vyb_instance_inject_status(vyb_instance* inst, uint32_t word) {
    if (!inst) return fail_invalid_program("Fix: pass a non-null instance.");
    std::lock_guard<std::mutex> ilk(inst->mu);
    cudaSetDevice(inst->dev->ordinal);
    // stream-ordered, like a kernel whose bounded wait ran out: the next submission on this instance reads it
    cudaError_t e = cudaMemcpyAsync(inst->status_dev, &word, 4, cudaMemcpyHostToDevice, inst->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(inst->stream);
    if (e != cudaSuccess) return fail_dispatch(int(e), "status injection failed: " + cuda_msg(e));
    clear_error();
    return VYB_OK;
}

int32_t vyb_submission_is_ready(const vyb_submission* s) {
    if (!s || s->consumed) return 0;
    return cudaEventQuery(s->done) == cudaSuccess ? 1 : 0;
}

int32_t vyb_submission_wait(vyb_submission* s, vyb_completion** completion) {
    if (!s || !completion) return fail_invalid_program("Fix: pass a non-null submission and completion out-pointer.");
    if (s->consumed) return fail_invalid_program("Fix: completion may be consumed only once.");
    vyb_instance* inst = s->inst;
    vyb_device* d = inst->dev;
    vyb_prepared* prep = s->prepared;
    cudaSetDevice(d->ordinal);
    cudaError_t e = cudaEventSynchronize(s->done);
    float ms = 0.0f;
    const bool timed = e == cudaSuccess && s->start && cudaEventElapsedTime(&ms, s->start, s->end) == cudaSuccess;
    // the status words this submission itself read back (never another submission's)
    const uint32_t status = e == cudaSuccess && s->status_host ? s->status_host[0] : 0;
    {
        std::lock_guard<std::mutex> ilk(inst->mu);
        for (void* t : s->temps) inst->release_temp(t);
        for (void* t : s->staged) inst->release_pinned(t);
        if (!prep && s->status_host) inst->release_pinned(s->status_host);
        if (!prep) {
            inst->release_event(s->start, true);
            inst->release_event(s->end, true);
            inst->release_event(s->done, false);
        }
    }
    if (!prep) {
        std::lock_guard<std::mutex> lk(d->mu);
        for (uint64_t id : s->resident_ids) {
            auto it = d->residents.find(id);
            if (it != d->residents.end() && it->second.inflight) it->second.inflight--;
        }
    }
    s->consumed = true;
    auto release_outputs = [&]() {
        std::lock_guard<std::mutex> ilk(inst->mu);
        if (prep) {
            prep->busy = false;
            return;
        }
        for (auto& o : s->outputs)
            if (o.host) inst->release_pinned(o.host);
    };
    if (e != cudaSuccess || status) {
        cudaGetLastError();
        release_outputs();
        delete s;
        // decide and word the failure while the device object is certainly alive: the submission may hold the last
        // reference to the instance, and the instance the last one to the device
        int32_t rc;
        const bool lost = e == cudaErrorIllegalAddress || e == cudaErrorLaunchFailure || e == cudaErrorHardwareStackError ||
                          e == cudaErrorIllegalInstruction || e == cudaErrorECCUncorrectable || e == cudaErrorDevicesUnavailable;
        if (e != cudaSuccess && lost) {
            vyb_device_mark_lost(d, cuda_msg(e).c_str());
            rc = fail_device_lost(d->device_name, d->generation.load(), cuda_msg(e));
        } else if (e != cudaSuccess) {
            rc = fail_dispatch(int(e), "submission failed: " + cuda_msg(e));
        } else {
            rc = fail_dispatch(int(status), "a bounded device-side wait ran out (kernel status word " +
                                                std::to_string(status) + "); the kernel drained without completing");
        }
        instance_unref(inst);
        return rc;
    }
    auto c = std::make_unique<vyb_completion>();
    c->inst = inst;
    c->prepared = prep;
    c->artifact = inst->artifact;
    c->outputs = prep ? prep->outputs : std::move(s->outputs);
    c->has_device_ns = timed;
    c->device_ns = timed ? uint64_t(double(ms) * 1.0e6) : 0;
    delete s;
    *completion = c.release();
    clear_error();
    return VYB_OK;
}

int32_t vyb_completion_output(const vyb_completion* c, uint32_t value_id, const uint8_t** bytes, size_t* len) {
    if (!c || !bytes || !len) return fail_invalid_program("Fix: pass non-null completion, bytes and len pointers.");
    for (const auto& o : c->outputs)
        if (o.value_id == value_id) {
            if (!o.host)
                return fail_invalid_program("Fix: output value " + std::to_string(value_id) +
                                            " was left resident (leave_resident=1); download it from its resident handle.");
            *bytes = static_cast<const uint8_t*>(o.host);
            *len = o.len;
            return VYB_OK;
        }
    return fail_invalid_program("Fix: value id " + std::to_string(value_id) + " is not an output of this artifact.");
}
uint32_t vyb_completion_output_count(const vyb_completion* c) { return c ? uint32_t(c->outputs.size()) : 0; }
int32_t vyb_completion_device_ns(const vyb_completion* c, uint64_t* ns) {
    if (!c || !ns) return fail_invalid_program("Fix: pass non-null completion and ns pointers.");
    if (!c->has_device_ns) return fail_unsupported("device timestamps for this submission");
    *ns = c->device_ns;
    return VYB_OK;
}
void vyb_completion_free(vyb_completion* c) {
    if (!c) return;
    {
        std::lock_guard<std::mutex> ilk(c->inst->mu);
        if (c->prepared) {
            c->prepared->busy = false;  // its buffers may be written by the next replay
        } else {
            for (auto& o : c->outputs)
                if (o.host) c->inst->release_pinned(o.host);
        }
    }
    instance_unref(c->inst);
    delete c;
}

// ---- prepared binding sets: one CUDA graph per set, one graph launch per submission ---------------------------------
constexpr size_t DIRECT_OUTPUT_BYTES = 256 * 1024;
int32_t vyb_prepare(vyb_instance* inst, const uint8_t artifact_digest[32], const vyb_binding* bindings, size_t n_bindings,
                    vyb_prepared** prepared) {
    if (!prepared) return fail_invalid_program("Fix: pass a non-null prepared out-pointer.");
    // one ordinary submission first: it validates the bindings exactly as vyb_submit does and runs every one-time
    // kernel configuration call outside stream capture
    {
        vyb_submission* sub = nullptr;
        if (int32_t rc = vyb_submit(inst, artifact_digest, bindings, n_bindings, nullptr, &sub)) return rc;
        vyb_completion* c = nullptr;
        if (int32_t rc = vyb_submission_wait(sub, &c)) return rc;
        vyb_completion_free(c);
    }
    vyb_device* d = inst->dev;
    const Program& p = inst->program;
    std::lock_guard<std::mutex> ilk(inst->mu);
    cudaSetDevice(d->ordinal);
    auto prep = std::make_unique<vyb_prepared>();
    prep->inst = inst;
    void* slot_ptr[16] = {nullptr};
    std::vector<std::pair<void*, size_t>> zero_fill;
    auto undo = [&]() {
        for (void* t : prep->temps) inst->release_temp(t);
        for (auto& in : prep->inputs) inst->release_pinned(in.staging);
        for (auto& o : prep->outputs)
            if (o.host) inst->release_pinned(o.host);
        if (prep->status_host) inst->release_pinned(prep->status_host);
        if (prep->done) inst->release_event(prep->done, false);
        std::lock_guard<std::mutex> lk(d->mu);
        for (uint64_t id : prep->resident_ids) {
            auto it = d->residents.find(id);
            if (it != d->residents.end() && it->second.inflight) it->second.inflight--;
        }
    };
    for (const BufferDecl& bd : p.buffers) {
        if (bd.access == VYB_ACCESS_WORKGROUP) continue;
        const size_t need = size_t(bd.count) * dtype_size_bytes(bd.dtype);
        const size_t logical = bd.has_output_byte_range ? size_t(bd.output_byte_end - bd.output_byte_begin) : need;
        const vyb_binding* b = nullptr;
        for (size_t i = 0; i < n_bindings; ++i)
            if (bindings[i].value_id == bd.binding) b = &bindings[i];
        const bool is_input = bd.access == VYB_ACCESS_READ_ONLY || bd.access == VYB_ACCESS_READ_WRITE;
        const bool is_output = bd.access == VYB_ACCESS_OUTPUT || bd.access == VYB_ACCESS_READ_WRITE;
        void* dev_ptr = nullptr;
        void* direct_host = nullptr;
        if (b && b->kind == VYB_BIND_RESIDENT) {
            std::lock_guard<std::mutex> lk(d->mu);
            Resident* r = nullptr;
            if (int32_t rc = d->resolve(b->resident, "CUDA resident dispatch", &r)) {
                undo();
                return rc;
            }
            r->inflight++;  // held for the life of the prepared set: the graph has the pointer baked in
            prep->resident_ids.push_back(b->resident.id);
            dev_ptr = r->ptr;
        } else if (!is_input && is_output && !bd.has_output_byte_range && need <= DIRECT_OUTPUT_BYTES &&
                   overwrites_every_output_byte(p) && p.kind != OpKind::LinearInt4Block) {  // whose residual add may run in place
            // A small output that its kernel writes completely: the kernel stores straight into mapped pinned host memory
            // (posted writes over PCIe, a few hundred transactions), which saves the device buffer and the copy node.
            direct_host = inst->acquire_pinned(need);
            if (!direct_host || cudaHostGetDevicePointer(&dev_ptr, direct_host, 0) != cudaSuccess) {
                cudaGetLastError();
                if (direct_host) inst->release_pinned(direct_host);
                undo();
                return fail_oom(need, 0);
            }
        } else {
            dev_ptr = inst->acquire_temp(need);
            if (!dev_ptr) {
                undo();
                return fail_oom(need, 0);
            }
            prep->temps.push_back(dev_ptr);
            if (is_input) {
                void* stage = inst->acquire_pinned(need);
                if (!stage) {
                    undo();
                    return fail_oom(need, 0);
                }
                std::memcpy(stage, b->host_ptr, need);
                prep->inputs.push_back({bd.binding, stage, need});
            } else if (!overwrites_every_output_byte(p)) {
                zero_fill.push_back({dev_ptr, need});
            }
        }
        slot_ptr[bd.binding] = dev_ptr;
        if (is_output) {
            OutputSlot o;
            o.value_id = bd.binding;
            o.dev_ptr = static_cast<uint8_t*>(dev_ptr) + (bd.has_output_byte_range ? bd.output_byte_begin : 0);
            o.len = logical;
            o.direct = direct_host != nullptr;
            o.host = direct_host ? direct_host : inst->acquire_pinned(logical);
            if (!o.host) {
                undo();
                return fail_oom(logical, 0);
            }
            prep->outputs.push_back(o);
        }
    }
    prep->status_host = static_cast<uint32_t*>(inst->acquire_pinned(16));
    prep->done = inst->acquire_event(false);
    if (!prep->status_host || !prep->done) {
        undo();
        return fail_oom(16, 0);
    }
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamBeginCapture(inst->stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
        for (auto& in : prep->inputs) {
            void* dst = slot_ptr[in.value_id];
            cudaMemcpyAsync(dst, in.staging, in.len, cudaMemcpyHostToDevice, inst->stream);
        }
        for (auto& z : zero_fill) cudaMemsetAsync(z.first, 0, z.second, inst->stream);
        // The kernels of a prepared set raise their status words straight in the set's own mapped pinned slot (they touch it
        // only when a bounded wait runs out), so the graph needs no status copy and no reset node: the host clears the
        // slot before every replay and reads it after the set's event.
        uint32_t* const shared_status = inst->status_dev;
        void* own_status = nullptr;
        if (cudaHostGetDevicePointer(&own_status, prep->status_host, 0) == cudaSuccess) inst->status_dev = static_cast<uint32_t*>(own_status);
        cudaError_t le = dispatch(inst, slot_ptr, inst->stream);
        inst->status_dev = shared_status;
        for (auto& o : prep->outputs)
            if (!o.direct) cudaMemcpyAsync(o.host, o.dev_ptr, o.len, cudaMemcpyDeviceToHost, inst->stream);
        if (!own_status) {
            cudaGetLastError();
            cudaMemcpyAsync(prep->status_host, inst->status_dev, 16, cudaMemcpyDeviceToHost, inst->stream);
            cudaMemsetAsync(inst->status_dev, 0, 16, inst->stream);
        }
        e = cudaStreamEndCapture(inst->stream, &graph);
        if (e == cudaSuccess && le != cudaSuccess) e = le;
    }
    if (e == cudaSuccess) e = cudaGraphInstantiate(&prep->exec, graph, 0);
    if (graph) cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        cudaGetLastError();
        undo();
        return fail_dispatch(int(e), "capturing the prepared submission failed: " + cuda_msg(e));
    }
    inst->refs.fetch_add(1);
    *prepared = prep.release();
    clear_error();
    return VYB_OK;
}

int32_t vyb_prepared_submit(vyb_prepared* prep, const vyb_binding* host_updates, size_t n_updates, vyb_submission** submission) {
    return vyb_prepared_submit_after(prep, nullptr, host_updates, n_updates, submission);
}

int32_t vyb_prepared_submit_after(vyb_prepared* prep, const vyb_submission* after, const vyb_binding* host_updates, size_t n_updates,
                                  vyb_submission** submission) {
    if (!prep || !submission || (!host_updates && n_updates))
        return fail_invalid_program("Fix: pass a non-null prepared set, updates and submission out-pointer.");
    vyb_instance* inst = prep->inst;
    vyb_device* d = inst->dev;
    if (after && (after->consumed || !after->done || after->inst->dev != d))
        return fail_invalid_program("Fix: `after` must be a pending submission (not yet waited for) on the same device.");
    if (int32_t rc = d->check_alive("submission")) return rc;
    if (inst->generation != d->generation.load())
        return fail_device_lost(d->device_name, inst->generation, "the instance belongs to a previous device generation");
    std::lock_guard<std::mutex> ilk(inst->mu);
    if (prep->busy)
        return fail_invalid_program(
            "Fix: the previous submission of this prepared set has not been waited for and freed; prepare one set per "
            "submission in flight.");
    for (size_t i = 0; i < n_updates; ++i) {
        const vyb_binding& b = host_updates[i];
        vyb_prepared::HostInput* in = nullptr;
        for (auto& cand : prep->inputs)
            if (cand.value_id == b.value_id) in = &cand;
        if (!in || b.kind != VYB_BIND_HOST)
            return fail_invalid_program("Fix: value id " + std::to_string(b.value_id) +
                                        " is not a host input of this prepared set; only host-bound inputs can be updated.");
        if (b.len != in->len || !b.host_ptr)
            return fail_invalid_program("Fix: host bytes for value id " + std::to_string(b.value_id) + " must be exactly " +
                                        std::to_string(in->len) + " bytes.");
        std::memcpy(in->staging, b.host_ptr, in->len);  // copied in, like a fresh BindingSet
    }
    cudaSetDevice(d->ordinal);
    std::memset(prep->status_host, 0, 16);
    cudaError_t e = cudaSuccess;
    // ordered behind another submission on the device: this instance's stream waits for that submission's completion event
    if (after && after->inst->stream != inst->stream) e = cudaStreamWaitEvent(inst->stream, after->done, 0);
    if (e == cudaSuccess) e = cudaGraphLaunch(prep->exec, inst->stream);
    if (e == cudaSuccess) e = cudaEventRecord(prep->done, inst->stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "replaying the prepared submission failed: " + cuda_msg(e));
    }
    prep->busy = true;
    auto sub = std::make_unique<vyb_submission>();
    sub->inst = inst;
    sub->prepared = prep;
    sub->done = prep->done;
    sub->status_host = prep->status_host;
    inst->refs.fetch_add(1);
    *submission = sub.release();
    clear_error();
    return VYB_OK;
}

int32_t vyb_prepared_free(vyb_prepared* prep) {
    if (!prep) return VYB_OK;
    vyb_instance* inst = prep->inst;
    vyb_device* d = inst->dev;
    {
        std::lock_guard<std::mutex> ilk(inst->mu);
        if (prep->busy)
            return fail_invalid_program("Fix: wait for and free the pending submission before freeing the prepared set.");
        cudaSetDevice(d->ordinal);
        if (prep->exec) cudaGraphExecDestroy(prep->exec);
        for (void* t : prep->temps) inst->release_temp(t);
        for (auto& in : prep->inputs) inst->release_pinned(in.staging);
        for (auto& o : prep->outputs)
            if (o.host) inst->release_pinned(o.host);
        inst->release_pinned(prep->status_host);
        inst->release_event(prep->done, false);
    }
    {
        std::lock_guard<std::mutex> lk(d->mu);
        for (uint64_t id : prep->resident_ids) {
            auto it = d->residents.find(id);
            if (it != d->residents.end() && it->second.inflight) it->second.inflight--;
        }
    }
    delete prep;
    instance_unref(inst);
    return VYB_OK;
}

// ---- kernel-level entry points ----------------------------------------------------------------------------------------------
int32_t vyb_k_int4_gemv_ex(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                           uint32_t n, uint32_t k, uint32_t group_size, uint32_t out_dtype, uint32_t flags,
                           void* stream, uint32_t* status) {
    if (!x_bf16 || !w_packed || !scale_bf16 || !y) return fail_invalid_program("Fix: pass non-null device pointers.");
    if (out_dtype != VYB_DT_BF16 && out_dtype != VYB_DT_F32)
        return fail_invalid_program("Fix: int4 gemv output dtype must be BF16 or F32.");
    if (!vybk::int4_gemv_supported(m, n, k, group_size))
        return fail_unsupported("int4 gemv shape m=" + std::to_string(m) + " n=" + std::to_string(n) + " k=" +
                                std::to_string(k) + " group=" + std::to_string(group_size) +
                                " (needs 1 <= m <= 8, group 128, k a multiple of 1024)");
    if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(w_packed) |
         reinterpret_cast<uintptr_t>(scale_bf16)) & 15)
        return fail_invalid_program("Fix: int4 gemv operands must be 16-byte aligned (bulk copies start on 16-byte boundaries).");
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "no usable CUDA device for the launch (" + cuda_msg(e) + "); there is no CPU path");
    }
    if ((flags & VYB_LAUNCH_LEAVE_ONE_SM) && sms > 1) --sms;  // room for a concurrent small kernel (the all-gather push)
    e = vybk::launch_int4_gemv(x_bf16, w_packed, scale_bf16, y, m, n, k, out_dtype == VYB_DT_F32 ? 1u : 0u, sms,
                               static_cast<cudaStream_t>(stream), status, (flags & VYB_LAUNCH_CONSTANT_WEIGHTS) != 0);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "int4 gemv launch failed: " + cuda_msg(e));
    }
    return VYB_OK;
}

namespace {
int32_t current_sm_count(int* sms) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "no usable CUDA device for the launch (" + cuda_msg(e) + "); there is no CPU path");
    }
    return VYB_OK;
}
int32_t launch_result(cudaError_t e, const char* what) {
    if (e == cudaErrorNotSupported) {
        cudaGetLastError();
        return fail_unsupported(std::string(what) + " with these dimensions");
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), std::string(what) + " launch failed: " + cuda_msg(e));
    }
    return VYB_OK;
}
}  // namespace

namespace {
int32_t to_gather(const vyb_allgather_ctx* ctx, vybk::PeerGather* ag) {
    if (!ctx) return fail_invalid_program("Fix: pass a non-null all-gather context.");
    if (ctx->world < 1 || ctx->world > 8 || ctx->rank >= ctx->world)
        return fail_invalid_program("Fix: the all-gather context needs 1 <= world <= 8 and rank < world, got world=" +
                                    std::to_string(ctx->world) + " rank=" + std::to_string(ctx->rank) + ".");
    if (!ctx->epoch) return fail_invalid_program("Fix: the all-gather context needs a local launch-counter word.");
    for (uint32_t r = 0; r < ctx->world; ++r)
        if (!ctx->peer_out[r] || !ctx->peer_flag[r])
            return fail_invalid_program("Fix: the all-gather context needs a gather buffer and an arrival counter for every rank.");
    ag->world = ctx->world;
    ag->rank = ctx->rank;
    for (int r = 0; r < 8; ++r) {
        ag->peer_out[r] = ctx->peer_out[r];
        ag->peer_flag[r] = ctx->peer_flag[r];
    }
    ag->epoch = ctx->epoch;
    ag->wait_clocks = ctx->wait_clocks;
    ag->slots = ctx->slots;
    return VYB_OK;
}
}  // namespace

int32_t vyb_k_allgather_push(const vyb_allgather_ctx* ctx, uint32_t half, uint32_t m, uint32_t n, void* stream,
                             uint32_t* status) {
    vybk::PeerGather ag;
    if (int32_t rc = to_gather(ctx, &ag)) return rc;
    if (half >= (ctx->slots ? ctx->slots : 2) || m == 0 || n == 0 || (uint64_t(m) * n) % 8)
        return fail_invalid_program("Fix: all-gather push needs a slot index below the context's slot count (two unless the "
                                    "context says otherwise) and m*n a multiple of 8 (16-byte stores).");
    return launch_result(vybk::launch_allgather_push(ag, half, m, n, static_cast<cudaStream_t>(stream), status),
                         "all-gather push");
}

int32_t vyb_k_int4_gemv_allgather(const vyb_allgather_ctx* ctx, uint32_t half, const void* x_bf16, const void* w_packed,
                                  const void* scale_bf16, uint32_t m, uint32_t n, uint32_t k, uint32_t group_size, uint32_t flags,
                                  void* stream, uint32_t* status) {
    vybk::PeerGather ag;
    if (int32_t rc = to_gather(ctx, &ag)) return rc;
    if (!x_bf16 || !w_packed || !scale_bf16) return fail_invalid_program("Fix: pass non-null device pointers.");
    if (half > 1) return fail_invalid_program("Fix: the gather buffer has two halves: pass half 0 or 1, alternating from launch to launch.");
    if (!vybk::int4_gemv_halfsm_supported(m, n, k, group_size))
        return fail_unsupported("gathering int4 gemv shape m=" + std::to_string(m) + " n=" + std::to_string(n) + " k=" +
                                std::to_string(k) + " group=" + std::to_string(group_size) +
                                " (needs 1 <= m <= 4, group 128, k 2048 or 4096)");
    if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(w_packed) | reinterpret_cast<uintptr_t>(scale_bf16)) & 15)
        return fail_invalid_program("Fix: int4 gemv operands must be 16-byte aligned.");
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "no usable CUDA device for the launch (" + cuda_msg(e) + "); there is no CPU path");
    }
    return launch_result(vybk::launch_int4_gemv_halfsm(x_bf16, w_packed, scale_bf16, nullptr, m, n, k, 0, sms,
                                                       static_cast<cudaStream_t>(stream), status,
                                                       (flags & VYB_LAUNCH_CONSTANT_WEIGHTS) != 0, &ag, half,
                                                       (flags & VYB_LAUNCH_PIPELINED_GATHER) != 0),
                         "gathering int4 gemv");
}

int32_t vyb_k_allgather_wait(const vyb_allgather_ctx* ctx, void* stream, uint32_t* status) {
    vybk::PeerGather ag;
    if (int32_t rc = to_gather(ctx, &ag)) return rc;
    return launch_result(vybk::launch_allgather_wait(ag, static_cast<cudaStream_t>(stream), status), "all-gather wait");
}

int32_t vyb_k_colpar_push(const vyb_allgather_ctx* ctx, const void* block, uint32_t rows, uint32_t row_bytes,
                          uint64_t dst_pitch_bytes, uint64_t dst_offset_bytes, void* stream, uint32_t* status) {
    vybk::PeerGather ag;
    if (int32_t rc = to_gather(ctx, &ag)) return rc;
    if (!block || (row_bytes | dst_pitch_bytes | dst_offset_bytes) % 16 || (reinterpret_cast<uintptr_t>(block) & 15))
        return fail_invalid_program("Fix: the column-parallel push needs a 16-byte aligned block and row bytes, pitch and "
                                    "offset that are multiples of 16 (16-byte stores).");
    // the tickets live behind the eight launch-counter words of the context's local block
    uint32_t* tickets = reinterpret_cast<uint32_t*>(ctx->epoch) + 8;
    return launch_result(vybk::launch_colpar_push(ag, block, rows, row_bytes, dst_pitch_bytes, dst_offset_bytes, tickets,
                                                  static_cast<cudaStream_t>(stream), status),
                         "column-parallel push");
}

int32_t vyb_k_int8_gemm_i32_gather(const vyb_allgather_ctx* ctx, const void* a_i8, const void* w_i8, uint32_t m, uint32_t n,
                                   uint32_t k, uint64_t dst_pitch_bytes, uint64_t dst_offset_bytes, void* stream,
                                   uint32_t* status) {
    vybk::PeerGather ag;
    if (int32_t rc = to_gather(ctx, &ag)) return rc;
    if (!a_i8 || !w_i8) return fail_invalid_program("Fix: pass non-null device pointers.");
    if ((dst_pitch_bytes | dst_offset_bytes) % 16 || n % 4)
        return fail_invalid_program("Fix: the gathering GEMM needs a pitch and an offset that are multiples of 16 bytes and n a "
                                    "multiple of 4 (16-byte stores into every rank's output).");
    if (!vybk::int8_gemm_pair_supported(m, n, k))
        return fail_unsupported("gathering int8 gemm shape m=" + std::to_string(m) + " n=" + std::to_string(n) + " k=" +
                                std::to_string(k) + " (needs m > 128, k a multiple of 16 and at most 132096); run "
                                "vyb_k_int8_gemm_i32 and vyb_k_colpar_push instead");
    if ((reinterpret_cast<uintptr_t>(a_i8) | reinterpret_cast<uintptr_t>(w_i8)) & 15)
        return fail_invalid_program("Fix: int8 gemm operands must be 16-byte aligned (TMA tensor maps need it).");
    int sms = 0;
    if (int32_t rc = current_sm_count(&sms)) return rc;
    vybk::GemmGatherOut go;
    go.count = ag.world;
    for (uint32_t r = 0; r < ag.world; ++r) go.dst[r] = ag.peer_out[r];
    go.pitch = dst_pitch_bytes / 4;
    go.col_off = dst_offset_bytes / 4;
    cudaError_t e = vybk::launch_int8_gemm_pair_gather(static_cast<const int8_t*>(a_i8), static_cast<const int8_t*>(w_i8), go, m, n,
                                                       k, sms, static_cast<cudaStream_t>(stream), status);
    if (e == cudaSuccess) e = vybk::launch_colpar_signal(ag, static_cast<cudaStream_t>(stream));
    return launch_result(e, "gathering int8 gemm");
}

int32_t vyb_k_colpar_wait(const vyb_allgather_ctx* ctx, uint32_t blocks, void* stream, uint32_t* status) {
    vybk::PeerGather ag;
    if (int32_t rc = to_gather(ctx, &ag)) return rc;
    return launch_result(vybk::launch_colpar_wait(ag, blocks, static_cast<cudaStream_t>(stream), status), "column-parallel wait");
}

int32_t vyb_k_tensor_peak(uint32_t int8, uint32_t iters, void* stream, uint32_t* status, double* ops_per_launch) {
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess)
        e = vybk::launch_tensor_peak(int8, iters, sms, static_cast<cudaStream_t>(stream), status, ops_per_launch);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "tensor peak launch failed: " + cuda_msg(e) + "; there is no CPU path");
    }
    return VYB_OK;
}

int32_t vyb_k_int4_gemv(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                        uint32_t n, uint32_t k, uint32_t group_size, uint32_t out_dtype, void* stream,
                        uint32_t* status) {
    return vyb_k_int4_gemv_ex(x_bf16, w_packed, scale_bf16, y, m, n, k, group_size, out_dtype, 0, stream, status);
}

// ---- the residual block around a decode projection, on raw device pointers --------------------------------------------
int32_t vyb_k_int4_linear_block(const void* x_bf16, const void* norm_weight_bf16, float norm_eps, const void* w_packed,
                                const void* scale_bf16, const void* gate_bf16, const void* residual_bf16, void* y_bf16, uint32_t m,
                                uint32_t n, uint32_t k, uint32_t group_size, uint32_t flags, void* stream, uint32_t* status) {
    if (!x_bf16 || !w_packed || !scale_bf16 || !y_bf16) return fail_invalid_program("Fix: pass non-null device pointers.");
    if (!norm_weight_bf16 && !residual_bf16 && !gate_bf16)
        return fail_invalid_program("Fix: pass a norm weight, a gate, a residual, or a norm weight with one of the two; vyb_k_int4_gemv is the bare projection.");
    if (gate_bf16 && residual_bf16) return fail_invalid_program("Fix: pass a gate or a residual behind the projection, not both.");
    const bool whole = m <= 2 && vybk::int4_gemv_halfsm_supported(m, n, k, group_size);
    const bool blocks = !norm_weight_bf16 && vybk::int4_gemv_kblocks_supported(m, n, k, group_size);
    if (!whole && !blocks)
        return fail_unsupported("int4 block gemv shape m=" + std::to_string(m) + " n=" + std::to_string(n) + " k=" + std::to_string(k) +
                                " group=" + std::to_string(group_size) +
                                " (needs group 128 and m <= 2 with k 2048 or 4096, or no norm with m <= 4 and k a larger multiple of 2048)");
    if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(w_packed) | reinterpret_cast<uintptr_t>(scale_bf16) |
         reinterpret_cast<uintptr_t>(norm_weight_bf16)) & 15)
        return fail_invalid_program("Fix: int4 gemv operands must be 16-byte aligned.");
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "no usable CUDA device for the launch (" + cuda_msg(e) + "); there is no CPU path");
    }
    const bool constant = (flags & VYB_LAUNCH_CONSTANT_WEIGHTS) != 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (whole)
        return launch_result(vybk::launch_int4_gemv_halfsm(x_bf16, w_packed, scale_bf16, y_bf16, m, n, k, 0, sms, s, status, constant,
                                                           nullptr, 0, false, norm_weight_bf16, norm_eps, residual_bf16, gate_bf16),
                             "int4 block gemv");
    bool fused = false;
    e = vybk::launch_int4_gemv_kblocks(x_bf16, w_packed, scale_bf16, y_bf16, m, n, k, 0, sms, s, constant, residual_bf16, gate_bf16, &fused);
    if (e == cudaSuccess && !fused)
        e = gate_bf16 ? vybk::launch_swiglu(gate_bf16, y_bf16, y_bf16, m * n, 1, s)
                      : vybk::launch_residual_add(residual_bf16, y_bf16, y_bf16, m * n, 1, s);
    return launch_result(e, "int4 block gemv");
}

namespace {
int32_t rt_float_dtype(uint32_t dtype, uint32_t* out) {
    if (dtype != VYB_DT_F32 && dtype != VYB_DT_BF16 && dtype != VYB_DT_F16)
        return fail_invalid_program("Fix: the element type must be F16, BF16, or F32.");
    *out = rt_dtype(dtype);
    return VYB_OK;
}
}  // namespace

int32_t vyb_k_rms_norm(const void* input, const void* weight, void* output, uint32_t rows, uint32_t hidden, float eps,
                       uint32_t dtype, void* stream) {
    uint32_t dt = 0;
    if (int32_t rc = rt_float_dtype(dtype, &dt)) return rc;
    if (!input || !weight || !output || rows == 0 || hidden == 0)
        return fail_invalid_program("Fix: pass non-null device pointers and nonzero rows and hidden size.");
    return launch_result(vybk::launch_rms_norm(input, weight, nullptr, output, rows, hidden, eps, dt, dt, hidden >= 2048,
                                               static_cast<cudaStream_t>(stream)),
                         "rms norm");
}
int32_t vyb_k_residual_add(const void* residual, const void* branch, void* output, uint32_t n, uint32_t dtype, void* stream) {
    uint32_t dt = 0;
    if (int32_t rc = rt_float_dtype(dtype, &dt)) return rc;
    if (!residual || !branch || !output || n == 0) return fail_invalid_program("Fix: pass non-null device pointers and n > 0.");
    return launch_result(vybk::launch_residual_add(residual, branch, output, n, dt, static_cast<cudaStream_t>(stream)), "residual add");
}
int32_t vyb_k_swiglu(const void* gate, const void* up, void* output, uint32_t n, uint32_t dtype, void* stream) {
    uint32_t dt = 0;
    if (int32_t rc = rt_float_dtype(dtype, &dt)) return rc;
    if (!gate || !up || !output || n == 0) return fail_invalid_program("Fix: pass non-null device pointers and n > 0.");
    return launch_result(vybk::launch_swiglu(gate, up, output, n, dt, static_cast<cudaStream_t>(stream)), "swiglu");
}

int32_t vyb_k_int4_prefill_gemm(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                uint32_t n, uint32_t k, uint32_t group_size, uint32_t out_dtype, void* stream,
                                uint32_t* status) {
    if (!x_bf16 || !w_packed || !scale_bf16 || !y) return fail_invalid_program("Fix: pass non-null device pointers.");
    if (out_dtype != VYB_DT_BF16 && out_dtype != VYB_DT_F32)
        return fail_invalid_program("Fix: int4 prefill output dtype must be BF16 or F32.");
    if (!vybk::int4_prefill_supported(m, n, k, group_size))
        return fail_unsupported("int4 prefill shape m=" + std::to_string(m) + " n=" + std::to_string(n) + " k=" +
                                std::to_string(k) + " group=" + std::to_string(group_size) +
                                " (needs k and group multiples of 64, group dividing k)");
    if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(w_packed) | reinterpret_cast<uintptr_t>(y)) & 15)
        return fail_invalid_program("Fix: int4 prefill operands must be 16-byte aligned (TMA tensor maps need it).");
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "no usable CUDA device for the launch (" + cuda_msg(e) + "); there is no CPU path");
    }
    e = vybk::launch_int4_prefill(x_bf16, w_packed, scale_bf16, y, m, n, k, group_size, out_dtype == VYB_DT_F32 ? 1u : 0u,
                                  sms, static_cast<cudaStream_t>(stream), status);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "int4 prefill launch failed: " + cuda_msg(e));
    }
    return VYB_OK;
}

int32_t vyb_k_quantize_per_token_int8(const void* x_bf16, void* q_i8, void* scales_f32, uint32_t m, uint32_t k,
                                      void* stream) {
    if (!x_bf16 || !q_i8 || !scales_f32) return fail_invalid_program("Fix: pass non-null device pointers.");
    if (m == 0 || k == 0) return fail_invalid_program("Fix: per-token quantisation requires nonzero m and k.");
    cudaError_t e = vybk::launch_quantize_per_token_int8(x_bf16, static_cast<int8_t*>(q_i8), static_cast<float*>(scales_f32),
                                                         m, k, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "per-token quantisation launch failed: " + cuda_msg(e));
    }
    return VYB_OK;
}


int32_t vyb_k_moe_route(const void* x_bf16, const void* w_router_bf16, void* routing_idx, void* routing_w, uint32_t tokens,
                        uint32_t hidden, uint32_t experts, uint32_t topk, void* stream) {
    if (!x_bf16 || !w_router_bf16 || !routing_idx || !routing_w) return fail_invalid_program("Fix: pass non-null device pointers.");
    return launch_result(vybk::launch_moe_route(x_bf16, w_router_bf16, static_cast<uint32_t*>(routing_idx),
                                                static_cast<float*>(routing_w), tokens, hidden, experts, topk,
                                                static_cast<cudaStream_t>(stream)),
                         "moe_route");
}

int32_t vyb_k_rows_gather_bf16(const void* src, const void* index_u32, void* dst, uint32_t rows, uint32_t row_elems,
                               void* stream) {
    if (rows && (!src || !index_u32 || !dst)) return fail_invalid_program("Fix: pass non-null device pointers.");
    int sms = 0;
    if (int32_t rc = current_sm_count(&sms)) return rc;
    return launch_result(vybk::launch_rows_gather_bf16(src, static_cast<const uint32_t*>(index_u32), dst, rows, row_elems, sms,
                                                       static_cast<cudaStream_t>(stream)),
                         "rows_gather_bf16");
}

int32_t vyb_k_moe_experts_int4(const void* x_sorted, const void* w13, const void* s13, const void* w2, const void* s2,
                               void* y_rows, void* h_scratch, const void* tile_expert_u32, const void* m_tiles_u32,
                               uint32_t max_rows, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t group_size,
                               void* stream, uint32_t* status) {
    if (!x_sorted || !w13 || !s13 || !w2 || !s2 || !y_rows || !h_scratch || !tile_expert_u32 || !m_tiles_u32)
        return fail_invalid_program("Fix: pass non-null device pointers.");
    int sms = 0;
    if (int32_t rc = current_sm_count(&sms)) return rc;
    return launch_result(
        vybk::launch_moe_experts_int4(x_sorted, w13, s13, w2, s2, y_rows, h_scratch, static_cast<const uint32_t*>(tile_expert_u32),
                                      static_cast<const uint32_t*>(m_tiles_u32), max_rows, hidden, inter, experts, group_size,
                                      sms, static_cast<cudaStream_t>(stream), status),
        "moe_experts_int4");
}

int32_t vyb_k_moe_combine(const void* y_rows, const void* pos_u32, const void* routing_w, void* out_bf16, uint32_t tokens,
                          uint32_t hidden, uint32_t topk, void* stream) {
    if (tokens && (!y_rows || !pos_u32 || !routing_w || !out_bf16)) return fail_invalid_program("Fix: pass non-null device pointers.");
    int sms = 0;
    if (int32_t rc = current_sm_count(&sms)) return rc;
    return launch_result(vybk::launch_moe_combine(y_rows, static_cast<const uint32_t*>(pos_u32),
                                                  static_cast<const float*>(routing_w), out_bf16, tokens, hidden, topk, sms,
                                                  static_cast<cudaStream_t>(stream)),
                         "moe_combine");
}

int32_t vyb_k_moe_ep_sizes(uint32_t tokens_local_max, uint32_t tokens_total, uint32_t hidden, uint32_t inter,
                           uint32_t experts, uint32_t topk, uint32_t world, vyb_moe_ep_ctx* ctx, uint64_t* symmetric_bytes,
                           uint64_t* local_bytes) {
    if (!ctx || !symmetric_bytes || !local_bytes) return fail_invalid_program("Fix: pass non-null out-pointers.");
    if (world < 1 || world > 8 || experts == 0 || experts % world || topk == 0 || tokens_total == 0 || tokens_local_max == 0)
        return fail_invalid_program("Fix: expert-parallel sizes need 1 <= world <= 8, experts divisible by world, nonzero tokens and topk.");
    vybk::MoeEp c;
    size_t total = 0;
    vybk::moe_ep_symmetric_layout(tokens_local_max, tokens_total, hidden, experts, topk, world, &c, &total);
    ctx->off_counts = c.off_counts;
    ctx->off_flags = c.off_flags;
    ctx->off_src = c.off_src;
    ctx->off_xg = c.off_xg;
    ctx->off_yhome = c.off_yhome;
    *symmetric_bytes = total;
    *local_bytes = vybk::moe_ep_local_bytes(tokens_local_max, tokens_total, hidden, inter, experts, topk, world);
    return VYB_OK;
}

int32_t vyb_k_moe_ep_ffn_int4(const vyb_moe_ep_ctx* ctx, const void* x_bf16, const void* w_router_bf16, const void* w13,
                              const void* s13, const void* w2, const void* s2, void* out_bf16, void* routing_idx,
                              void* routing_w, void* local_scratch, uint32_t tokens, uint32_t tokens_total, uint32_t hidden,
                              uint32_t inter, uint32_t experts, uint32_t topk, uint32_t group_size, void* stream,
                              uint32_t* status) {
    if (!ctx || !x_bf16 || !w_router_bf16 || !w13 || !s13 || !w2 || !s2 || !out_bf16 || !routing_idx || !routing_w || !local_scratch)
        return fail_invalid_program("Fix: pass non-null device pointers and context.");
    if (ctx->world < 1 || ctx->world > 8 || ctx->rank >= ctx->world)
        return fail_invalid_program("Fix: the expert-parallel context needs 1 <= world <= 8 and rank < world.");
    vybk::MoeEp c;
    c.world = ctx->world;
    c.rank = ctx->rank;
    for (uint32_t r = 0; r < 8; ++r) c.peer_base[r] = ctx->peer_base[r];
    for (uint32_t r = 0; r < ctx->world; ++r)
        if (!c.peer_base[r]) return fail_invalid_program("Fix: the expert-parallel context needs the symmetric region of every rank.");
    c.off_counts = ctx->off_counts;
    c.off_flags = ctx->off_flags;
    c.off_src = ctx->off_src;
    c.off_xg = ctx->off_xg;
    c.off_yhome = ctx->off_yhome;
    c.wait_clocks = ctx->wait_clocks;
    int sms = 0;
    if (int32_t rc = current_sm_count(&sms)) return rc;
    return launch_result(vybk::launch_moe_ep_ffn(c, x_bf16, w_router_bf16, w13, s13, w2, s2, out_bf16,
                                                 static_cast<uint32_t*>(routing_idx), static_cast<float*>(routing_w),
                                                 local_scratch, tokens, tokens_total, hidden, inter, experts, topk, group_size,
                                                 sms, static_cast<cudaStream_t>(stream), status),
                         "expert-parallel moe_ffn_int4");
}

int32_t vyb_k_moe_ffn_int4_scratch_bytes(uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts,
                                         uint32_t topk, uint64_t* bytes) {
    if (!bytes) return fail_invalid_program("Fix: pass a non-null byte-count out-pointer.");
    *bytes = vybk::moe_ffn_int4_scratch_bytes(tokens, hidden, inter, experts, topk);
    return VYB_OK;
}

int32_t vyb_k_moe_ffn_int4(const void* x_bf16, const void* w_router_bf16, const void* w13, const void* s13, const void* w2,
                           const void* s2, void* out_bf16, void* routing_idx, void* routing_w, void* scratch,
                           uint64_t scratch_bytes, uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts,
                           uint32_t topk, uint32_t group_size, void* stream, uint32_t* status) {
    if (!x_bf16 || !w_router_bf16 || !w13 || !s13 || !w2 || !s2 || !out_bf16 || !routing_idx || !routing_w || !scratch)
        return fail_invalid_program("Fix: pass non-null device pointers.");
    if (!vybk::moe_ffn_int4_supported(tokens, hidden, inter, experts, topk, group_size))
        return fail_unsupported("moe_ffn_int4 shape hidden=" + std::to_string(hidden) + " inter=" + std::to_string(inter) +
                                " experts=" + std::to_string(experts) + " topk=" + std::to_string(topk) +
                                " (needs hidden and inter multiples of 256, group a multiple of 64, experts <= 64, topk <= 8)");
    const uint64_t need = vybk::moe_ffn_int4_scratch_bytes(tokens, hidden, inter, experts, topk);
    if (scratch_bytes < need)
        return fail_invalid_program("Fix: moe_ffn_int4 needs " + std::to_string(need) + " scratch bytes, got " +
                                    std::to_string(scratch_bytes) + " (ask vyb_k_moe_ffn_int4_scratch_bytes).");
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "no usable CUDA device for the launch (" + cuda_msg(e) + "); there is no CPU path");
    }
    e = vybk::launch_moe_ffn_int4(x_bf16, w_router_bf16, w13, s13, w2, s2, out_bf16, static_cast<uint32_t*>(routing_idx),
                                  static_cast<float*>(routing_w), scratch, tokens, hidden, inter, experts, topk, group_size,
                                  sms, static_cast<cudaStream_t>(stream), status);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "moe_ffn_int4 launch failed: " + cuda_msg(e));
    }
    return VYB_OK;
}

int32_t vyb_k_int8_gemm_i32(const void* a_i8, const void* w_i8, void* out_i32, uint32_t m, uint32_t n, uint32_t k,
                            void* stream, uint32_t* status) {
    return vyb_k_int8_gemm_i32_ex(a_i8, w_i8, out_i32, m, n, k, 0, stream, status);
}

int32_t vyb_k_int8_gemm_i32_ex(const void* a_i8, const void* w_i8, void* out_i32, uint32_t m, uint32_t n, uint32_t k,
                               uint32_t flags, void* stream, uint32_t* status) {
    if (!a_i8 || !w_i8 || !out_i32) return fail_invalid_program("Fix: pass non-null device pointers.");
    if (!vybk::int8_gemm_supported(m, n, k))
        return fail_unsupported("int8 gemm shape m=" + std::to_string(m) + " n=" + std::to_string(n) + " k=" +
                                std::to_string(k) + " (needs k a multiple of 16 and at most 132096)");
    if ((reinterpret_cast<uintptr_t>(a_i8) | reinterpret_cast<uintptr_t>(w_i8) | reinterpret_cast<uintptr_t>(out_i32)) & 15)
        return fail_invalid_program("Fix: int8 gemm operands must be 16-byte aligned (TMA tensor maps need it).");
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "no usable CUDA device for the launch (" + cuda_msg(e) + "); there is no CPU path");
    }
    if ((flags & VYB_LAUNCH_LEAVE_COPY_SMS) && sms > 32) sms -= 16;  // room for a concurrent copy kernel (the peer-store gather)
    e = vybk::launch_int8_gemm(static_cast<const int8_t*>(a_i8), static_cast<const int8_t*>(w_i8),
                               static_cast<int32_t*>(out_i32), m, n, k, sms, static_cast<cudaStream_t>(stream), status);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "int8 gemm launch failed: " + cuda_msg(e));
    }
    return VYB_OK;
}

int32_t vyb_k_int8_weight_only_linear(const void* x_f32, const void* w_i8, const void* scale_f32, void* y_f32,
                                      uint32_t m, uint32_t n, uint32_t k, void* stream) {
    if (!x_f32 || !w_i8 || !scale_f32 || !y_f32) return fail_invalid_program("Fix: pass non-null device pointers.");
    if (m == 0 || n == 0 || k == 0)
        return fail_invalid_program("Fix: int8 weight-only linear requires nonzero m, n and k.");
    cudaError_t e = vybk::launch_int8_weight_only_linear(static_cast<const float*>(x_f32), static_cast<const int8_t*>(w_i8),
                                                         static_cast<const float*>(scale_f32), static_cast<float*>(y_f32),
                                                         m, n, k, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), "int8 weight-only launch failed: " + cuda_msg(e));
    }
    return VYB_OK;
}

}  // extern "C"
