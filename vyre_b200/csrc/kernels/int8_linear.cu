// int8 weight-only linear:  y[m, n] = sum_k x[m, k] * (f32(w[n, k]) * s[n]),  x/y f32, w int8 [n, k].
//
// At the benchmark size (16 x 1024 x 1024, 1.2 MB of traffic) the op is launch-latency bound, so the
// kernel is kept simple and wide: one warp per output channel streams its weight row once with 128-bit loads
// (16 weights per lane per step), keeps up to 16 batch accumulators in registers, and reduces them with warp
// shuffles. The per-channel scale is applied once to the reduced sum. Larger batches loop in blocks of 16.
//
// Composition of vyre-libs/src/nn/quant/int8.rs:15-50 (int8_unpack, here on signed bytes packed four per
// word instead of one per word) and vyre-libs/src/nn/linear/inner/builder.rs:241
// (linear_rows_no_bias_out_in, f32 accumulate).
#include <atomic>

#include "kernels.h"

namespace vybk {
namespace {

constexpr int MB = 16;  // batch rows held in registers

__global__ void __launch_bounds__(256) int8_weight_only_kernel(const float* __restrict__ x,
                                                              const int8_t* __restrict__ w,
                                                              const float* __restrict__ scale, float* __restrict__ y,
                                                              uint32_t m, uint32_t n, uint32_t k) {
    const uint32_t col = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (col >= n) return;
    const int8_t* wr = w + size_t(col) * k;
    const bool vec_ok = (k % 16 == 0) && (((reinterpret_cast<uintptr_t>(wr) | reinterpret_cast<uintptr_t>(x)) & 15) == 0);
    for (uint32_t m0 = 0; m0 < m; m0 += MB) {
        float acc[MB];
#pragma unroll
        for (int j = 0; j < MB; ++j) acc[j] = 0.0f;
        if (vec_ok) {
            for (uint32_t k0 = lane * 16; k0 < k; k0 += 32 * 16) {
                const int4 pk = *reinterpret_cast<const int4*>(wr + k0);
                const int words[4] = {pk.x, pk.y, pk.z, pk.w};
                float wf[16];
#pragma unroll
                for (int q = 0; q < 4; ++q)
#pragma unroll
                    for (int b = 0; b < 4; ++b) wf[q * 4 + b] = float(int8_t((words[q] >> (8 * b)) & 0xFF));
#pragma unroll
                for (int j = 0; j < MB; ++j) {
                    if (m0 + j < m) {
                        const float4* xr = reinterpret_cast<const float4*>(x + size_t(m0 + j) * k + k0);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 xv = xr[q];
                            acc[j] = fmaf(xv.x, wf[q * 4 + 0], acc[j]);
                            acc[j] = fmaf(xv.y, wf[q * 4 + 1], acc[j]);
                            acc[j] = fmaf(xv.z, wf[q * 4 + 2], acc[j]);
                            acc[j] = fmaf(xv.w, wf[q * 4 + 3], acc[j]);
                        }
                    }
                }
            }
        } else {
            for (uint32_t kk = lane; kk < k; kk += 32) {
                const float wv = float(wr[kk]);
#pragma unroll
                for (int j = 0; j < MB; ++j)
                    if (m0 + j < m) acc[j] = fmaf(x[size_t(m0 + j) * k + kk], wv, acc[j]);
            }
        }
        const float s = scale[col];
#pragma unroll
        for (int j = 0; j < MB; ++j) {
            float v = acc[j];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m0 + j < m) y[size_t(m0 + j) * n + col] = v * s;
        }
    }
}

// The same operator with the activations staged in shared memory: every warp of the kernel above streams all sixteen
// activation rows through L1 for its one output channel (64 KB per warp, 64 MB per launch at the benchmark size, which is
// what its time goes to). Here a block of four warps loads a 16-row x 1024-k activation tile once, each warp owns TWO
// output channels (an activation register feeds two weights), a lane takes four consecutive k per step so that the
// float4 reads of a warp are conflict-free and its weight reads are one 128-byte line per channel.
constexpr int KC = 1024;   // k per shared-memory tile
constexpr int CPW = 2;     // output channels per warp
constexpr int WPB = 4;     // warps per block
__global__ void __launch_bounds__(WPB * 32) int8_weight_only_tiled_kernel(const float* __restrict__ x, const int8_t* __restrict__ w,
                                                                          const float* __restrict__ scale, float* __restrict__ y,
                                                                          uint32_t m, uint32_t n, uint32_t k) {
    extern __shared__ __align__(16) float xs[];  // [MB][KC]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t col0 = (blockIdx.x * WPB + warp) * CPW;
    for (uint32_t m0 = 0; m0 < m; m0 += MB) {
        float acc[MB][CPW];
#pragma unroll
        for (int j = 0; j < MB; ++j)
#pragma unroll
            for (int c = 0; c < CPW; ++c) acc[j][c] = 0.0f;
        for (uint32_t kc = 0; kc < k; kc += KC) {
            const uint32_t klen = min(uint32_t(KC), k - kc);  // a multiple of 4
            __syncthreads();
            for (uint32_t i = threadIdx.x; i < MB * (KC / 4); i += WPB * 32) {
                const uint32_t j = i / (KC / 4), q = (i % (KC / 4)) * 4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (m0 + j < m && q < klen) v = *reinterpret_cast<const float4*>(x + size_t(m0 + j) * k + kc + q);
                *reinterpret_cast<float4*>(xs + j * KC + q) = v;
            }
            __syncthreads();
            for (uint32_t q = lane * 4; q < klen; q += 128) {
                float wf[CPW][4];
#pragma unroll
                for (int c = 0; c < CPW; ++c) {
                    int word = 0;
                    if (col0 + c < n) word = *reinterpret_cast<const int*>(w + size_t(col0 + c) * k + kc + q);
#pragma unroll
                    for (int b = 0; b < 4; ++b) wf[c][b] = float(int8_t((word >> (8 * b)) & 0xFF));
                }
#pragma unroll
                for (int j = 0; j < MB; ++j) {
                    const float4 xv = *reinterpret_cast<const float4*>(xs + j * KC + q);
#pragma unroll
                    for (int c = 0; c < CPW; ++c) {
                        acc[j][c] = fmaf(xv.x, wf[c][0], acc[j][c]);
                        acc[j][c] = fmaf(xv.y, wf[c][1], acc[j][c]);
                        acc[j][c] = fmaf(xv.z, wf[c][2], acc[j][c]);
                        acc[j][c] = fmaf(xv.w, wf[c][3], acc[j][c]);
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < CPW; ++c) {
            const float s = col0 + c < n ? scale[col0 + c] : 0.0f;
#pragma unroll
            for (int j = 0; j < MB; ++j) {
                float v = acc[j][c];
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0 && m0 + j < m && col0 + c < n) y[size_t(m0 + j) * n + col0 + c] = v * s;
            }
        }
    }
}

}  // namespace

cudaError_t launch_int8_weight_only_linear(const float* x, const int8_t* w, const float* scale, float* y, uint32_t m,
                                           uint32_t n, uint32_t k, cudaStream_t stream) {
    // k a multiple of 4 and 16-byte aligned operands: the shared-memory form; anything else: a warp per channel from L1
    if (k % 4 == 0 && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
        static std::atomic<uint64_t> configured{0};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const uint64_t bit = 1ull << (dev & 63);
        constexpr int SMEM = MB * KC * 4;
        if (!(configured.load(std::memory_order_acquire) & bit)) {
            e = cudaFuncSetAttribute(int8_weight_only_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
            if (e != cudaSuccess) return e;
            configured.fetch_or(bit, std::memory_order_release);
        }
        const uint32_t per_block = WPB * CPW;
        int8_weight_only_tiled_kernel<<<(n + per_block - 1) / per_block, WPB * 32, SMEM, stream>>>(x, w, scale, y, m, n, k);
        return cudaGetLastError();
    }
    int8_weight_only_kernel<<<(n + 7) / 8, 256, 0, stream>>>(x, w, scale, y, m, n, k);
    return cudaGetLastError();
}

}  // namespace vybk
