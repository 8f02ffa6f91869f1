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

}  // namespace

cudaError_t launch_int8_weight_only_linear(const float* x, const int8_t* w, const float* scale, float* y, uint32_t m,
                                           uint32_t n, uint32_t k, cudaStream_t stream) {
    int8_weight_only_kernel<<<(n + 7) / 8, 256, 0, stream>>>(x, w, scale, y, m, n, k);
    return cudaGetLastError();
}

}  // namespace vybk
