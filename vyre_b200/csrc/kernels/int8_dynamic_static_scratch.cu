// Dynamic int8 linear whose scratch lives in a fixed device array instead of an allocation.
//
//   x_scale[t] = max|x[t,:]| / 127,  xq = clamp(rint(x / x_scale), -127, 127),  y int32 [m,n] = xq . w^T
//
// The regular path keeps the quantised activations `xq` in a buffer that the instance allocates when it is
// materialised. Some callers may not allocate at all once they are running: a serving loop that has handed every
// free byte of device memory to its cache and pinned the rest, a host thread inside a region where the allocator's
// lock must not be taken, or a library embedded in a process whose memory budget was fixed at start-up. For them
// this file offers the same two kernels (per-token quantiser, then the tcgen05 int8 GEMM) with `xq` placed in a
// file-scope device array of fixed size. The array belongs to the module that holds these kernels: the device
// memory for it is reserved when that module is loaded on a device, which with lazy module loading happens during
// the first, set-up call on that device (see below) and never after it.
//
// Rules that follow from sharing one array:
//   * m * k must not exceed STATIC_SCRATCH_BYTES (8 MiB); larger shapes are refused before anything is launched.
//   * Every call on a device uses the same array. The quantiser overwrites every byte the GEMM of the same call
//     reads, so nothing has to start at zero and nothing is cleared. Two calls whose work overlaps in time (two
//     streams, or two host threads) race on the array and produce garbage; callers serialise them on one stream.
//   * The first call on each device resolves the array's device address (a symbol lookup in the loaded module).
//     That lookup is set-up work: make the first call during initialisation, before any stream capture begins.
#include <atomic>
#include <mutex>

#include <string>

#include "../host/model.hpp"
#include "kernels.h"

namespace vybk {
namespace {

constexpr size_t STATIC_SCRATCH_BYTES = size_t(8) << 20;
constexpr int MAX_DEVICES = 64;

static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

std::mutex g_setup_mutex;
std::atomic<int8_t*> g_scratch_ptr[MAX_DEVICES];

// The device address of the array on the current device; resolved once per device, with that device current.
cudaError_t static_scratch_for_current_device(int8_t** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
    int8_t* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        p = g_scratch_ptr[dev].load(std::memory_order_acquire);
        if (!p) {
            void* sym = nullptr;
            e = cudaGetSymbolAddress(&sym, g_static_scratch);
            if (e != cudaSuccess) return e;
            if (!sym) return cudaErrorInvalidSymbol;
            p = static_cast<int8_t*>(sym);
            g_scratch_ptr[dev].store(p, std::memory_order_release);
        }
    }
    *out = p;
    return cudaSuccess;
}

}  // namespace

size_t int8_dynamic_static_scratch_limit() { return STATIC_SCRATCH_BYTES; }

cudaError_t launch_int8_dynamic_static_scratch(const void* x_bf16, const int8_t* w, float* x_scale, int32_t* y,
                                               uint32_t m, uint32_t n, uint32_t k, int sm_count, cudaStream_t stream,
                                               uint32_t* status) {
    if (size_t(m) * size_t(k) > STATIC_SCRATCH_BYTES) return cudaErrorInvalidValue;
    int8_t* xq = nullptr;
    cudaError_t e = static_scratch_for_current_device(&xq);
    if (e != cudaSuccess) return e;
    e = launch_quantize_per_token_int8(x_bf16, xq, x_scale, m, k, stream);
    if (e != cudaSuccess) return e;
    return launch_int8_gemm(xq, w, y, m, n, k, sm_count, stream, status);
}

}  // namespace vybk

// C-ABI entry point (declared in include/vyre_b200.h). Same operands and results as vyb_k_quantize_per_token_int8
// followed by vyb_k_int8_gemm_i32, minus the caller-provided buffer for the quantised activations.
extern "C" int32_t vyb_k_linear_int8_dynamic_static_scratch(const void* x_bf16, const void* w_i8, void* x_scale_f32,
                                                            void* y_i32, uint32_t m, uint32_t n, uint32_t k,
                                                            void* stream, uint32_t* status) {
    using namespace vyb;
    if (!x_bf16 || !w_i8 || !x_scale_f32 || !y_i32) return fail_invalid_program("Fix: pass non-null device pointers.");
    if (m == 0 || n == 0 || k == 0) return fail_invalid_program("Fix: the dynamic int8 linear requires nonzero m, n and k.");
    const size_t limit = vybk::int8_dynamic_static_scratch_limit();
    if (size_t(m) * size_t(k) > limit)
        return fail_invalid_program("the quantised activations need " + std::to_string(size_t(m) * size_t(k)) +
                                    " bytes but the fixed scratch array holds " + std::to_string(limit) +
                                    ". Fix: split the batch so that m * k <= " + std::to_string(limit) +
                                    ", or use vyb_k_quantize_per_token_int8 + vyb_k_int8_gemm_i32 with your own buffer.");
    if (!vybk::int8_gemm_supported(m, n, k))
        return fail_unsupported("int8 gemm shape m=" + std::to_string(m) + " n=" + std::to_string(n) + " k=" +
                                std::to_string(k) + " (needs k a multiple of 16 and at most 132096)");
    if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(w_i8) | reinterpret_cast<uintptr_t>(y_i32)) & 15)
        return fail_invalid_program("Fix: dynamic int8 linear operands must be 16-byte aligned (TMA tensor maps need it).");
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), std::string("no usable CUDA device for the launch (") + cudaGetErrorName(e) +
                                         "); there is no CPU path");
    }
    e = vybk::launch_int8_dynamic_static_scratch(x_bf16, static_cast<const int8_t*>(w_i8), static_cast<float*>(x_scale_f32),
                                                 static_cast<int32_t*>(y_i32), m, n, k, sms,
                                                 static_cast<cudaStream_t>(stream), status);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail_dispatch(int(e), std::string("dynamic int8 linear (fixed scratch) failed: ") + cudaGetErrorName(e) + ": " +
                                         cudaGetErrorString(e));
    }
    return VYB_OK;
}
