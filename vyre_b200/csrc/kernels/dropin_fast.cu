// Fast kernels behind the reference's OWN operators and layouts (large shapes; small ones keep the reference-order
// kernels of ref_ops.cu, which are bit-exact against the reference interpreter):
//
//  * vyre-libs::nn::linear_4bit_affine_grouped (vyre-libs/src/nn/linear/inner/linear_4bit.rs:357-775):
//      out[b, i] = bias[i] + sum_k x[b, k] * fma(f32(nibble), s, -zp * s)
//    with the reference's layout untouched: words w[(k / 8) * N + i] (8 nibbles each, nibble k % 8 at bit 4 (k % 8)),
//    f32 scale and u32 zero point sidecars [group][N], f32 activations, f32 output. The reference kernel gives one
//    warp to every output and strides its lanes over k, which makes every weight load a 4-byte access with stride N.
//    That layout is made for the opposite assignment: for a fixed k-block consecutive OUTPUTS are contiguous. Here a
//    thread owns one output (a warp reads 128 contiguous bytes of W per k-block), keeps up to eight batch rows of
//    accumulators (every weight is dequantised once and used eight times), reads activations from shared memory as
//    broadcast float4s, and the block splits k over threadIdx.y when there are too few outputs to fill the GPU.
//  * vyre-primitives i4x8_[batched_]matvec_f32_scaled (vyre-primitives/src/math/quantized/programs.rs:186-300, body
//    program_helpers.rs:7-81): out[b, r] = scale[r] * sum_c s4(w[r, c]) * x[b, c], signed two's-complement nibbles,
//    row-major words. The reference gives a thread to every (batch, row) and walks the row serially; here a warp owns
//    a row (coalesced 128-byte loads), eight batch rows share every weight, lanes fold by shuffles.
//
// Both sum in a different order than the reference (which is lane-strided then folded, or strictly sequential), so
// results agree with it bit for bit only where the sums are exact (the reference's dyadic sweep) and otherwise within
// its own drift window for this operator (LINEAR_4BIT_AFFINE_GROUPED_OUTPUT_DRIFT_ABS_TOLERANCE = 1e-4 scaled to the
// output magnitude). The per-weight dequantisation is the reference's exact expression.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "kernels.h"

namespace vybk {
namespace {

constexpr int MV_BT = 8;     // batch rows per block of the matvec kernel

// Block: TX x KS threads. Thread (tx, ty) owns OT outputs (i = block base + tx + o * TX: for a fixed o a warp reads 128
// contiguous bytes of one k-block row of W) and the ty-th run of consecutive words of every KCHUNK-deep chunk of k.
// BT batch rows share every dequantised weight; BT * KCHUNK activations (16 KB) are staged per chunk, so few batch rows
// mean deep chunks and many weight words in flight per thread. The words of the NEXT chunk are loaded into registers
// before this chunk's barrier, so the global loads overlap the staging of x and the arithmetic.
// grid (ceil(N / (TX * OT)), ceil(B / BT)).
template <int TX, int OT, int KS, int BT, int KCHUNK>
__global__ void __launch_bounds__(TX* KS) affine_grouped_fast_kernel(const float* __restrict__ x, const uint32_t* __restrict__ w,
                                                                      const float* __restrict__ scale,
                                                                      const uint32_t* __restrict__ zp,
                                                                      const float* __restrict__ bias, float* __restrict__ out,
                                                                      uint32_t in_dim, uint32_t out_dim, uint32_t group,
                                                                      int group_shift, uint32_t batch) {
    constexpr int WPT = (KCHUNK / 8) / KS;
    constexpr int XS = BT * KCHUNK, RED = KS * BT * OT * TX;
    __shared__ __align__(16) float smem[XS > RED ? XS : RED];
    float(*xs)[KCHUNK] = reinterpret_cast<float(*)[KCHUNK]>(smem);
    const uint32_t tx = threadIdx.x, ty = threadIdx.y;
    const uint32_t i0 = blockIdx.x * (TX * OT) + tx;
    const uint32_t b0 = blockIdx.y * BT;
    const uint32_t nb = min(uint32_t(BT), batch - b0);
    const uint32_t words = in_dim / 8;
    float acc[BT][OT];
#pragma unroll
    for (int b = 0; b < BT; ++b)
#pragma unroll
        for (int o = 0; o < OT; ++o) acc[b][o] = 0.0f;
    uint32_t wcur[WPT][OT], wnext[WPT][OT];
    auto fetch = [&](uint32_t (&dst)[WPT][OT], uint32_t k0) {
#pragma unroll
        for (int j = 0; j < WPT; ++j) {
            const uint32_t kw = k0 / 8 + ty * WPT + j;
#pragma unroll
            for (int o = 0; o < OT; ++o) {
                const uint32_t i = i0 + o * TX;
                dst[j][o] = (kw < words && i < out_dim) ? __ldg(w + size_t(kw) * out_dim + i) : 0u;
            }
        }
    };
    fetch(wcur, 0);
    uint32_t cur_group = 0xFFFFFFFFu;
    float s[OT], zero_off[OT];
#pragma unroll
    for (int o = 0; o < OT; ++o) s[o] = zero_off[o] = 0.0f;
    for (uint32_t k0 = 0; k0 < in_dim; k0 += KCHUNK) {
        const uint32_t kc = min(uint32_t(KCHUNK), in_dim - k0);
        fetch(wnext, k0 + KCHUNK);  // past the end: zeros, never used
        __syncthreads();
        for (uint32_t e = ty * TX + tx; e < BT * (KCHUNK / 4); e += TX * KS) {  // float4 per thread; in_dim % 8 == 0
            const uint32_t b = e / (KCHUNK / 4), k = (e % (KCHUNK / 4)) * 4;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (b < nb && k < kc) v = __ldg(reinterpret_cast<const float4*>(x + size_t(b0 + b) * in_dim + k0 + k));
            *reinterpret_cast<float4*>(&xs[b][k]) = v;
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < WPT; ++j) {
            const uint32_t wi = ty * WPT + j;  // same for the whole warp
            if (wi * 8 < kc) {
                const uint32_t k = k0 + wi * 8;
                const uint32_t g = group_shift >= 0 ? (k >> group_shift) : k / group;
                if (g != cur_group) {  // group % 8 == 0: a word never straddles two groups
                    cur_group = g;
#pragma unroll
                    for (int o = 0; o < OT; ++o) {
                        const uint32_t i = min(i0 + o * TX, out_dim - 1);
                        s[o] = scale[size_t(g) * out_dim + i];
                        zero_off[o] = __fmaf_rn(float(zp[size_t(g) * out_dim + i]), __fmaf_rn(-1.0f, s[o], -0.0f), -0.0f);
                    }
                }
                float wv[OT][8];
#pragma unroll
                for (int o = 0; o < OT; ++o) {
                    const uint32_t lo = wcur[j][o] & 0x0F0F0F0Fu, hi = (wcur[j][o] >> 4) & 0x0F0F0F0Fu;  // nibbles 0,2,4,6 / 1,3,5,7
#pragma unroll
                    for (int n = 0; n < 4; ++n) {
                        // f32(nibble) without the conversion unit: 0x4B0000nn is 2^23 + nn, and the subtraction is exact
                        const float even = __fsub_rn(__uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7540 + n)), 8388608.0f);
                        const float odd = __fsub_rn(__uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7540 + n)), 8388608.0f);
                        wv[o][2 * n] = __fmaf_rn(even, s[o], zero_off[o]);
                        wv[o][2 * n + 1] = __fmaf_rn(odd, s[o], zero_off[o]);
                    }
                }
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    const float4 xa = *reinterpret_cast<const float4*>(&xs[b][wi * 8]);
                    const float4 xb = *reinterpret_cast<const float4*>(&xs[b][wi * 8 + 4]);
#pragma unroll
                    for (int o = 0; o < OT; ++o) {
                        float a = acc[b][o];
                        a = __fmaf_rn(xa.x, wv[o][0], a);
                        a = __fmaf_rn(xa.y, wv[o][1], a);
                        a = __fmaf_rn(xa.z, wv[o][2], a);
                        a = __fmaf_rn(xa.w, wv[o][3], a);
                        a = __fmaf_rn(xb.x, wv[o][4], a);
                        a = __fmaf_rn(xb.y, wv[o][5], a);
                        a = __fmaf_rn(xb.z, wv[o][6], a);
                        a = __fmaf_rn(xb.w, wv[o][7], a);
                        acc[b][o] = a;
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < WPT; ++j)
#pragma unroll
            for (int o = 0; o < OT; ++o) wcur[j][o] = wnext[j][o];
    }
    // fold the k-slices in a fixed order (deterministic), every thread takes its share of the batch rows
    __syncthreads();
    float* red = smem;  // [KS][BT][OT * TX]
#pragma unroll
    for (int b = 0; b < BT; ++b)
#pragma unroll
        for (int o = 0; o < OT; ++o) red[(ty * BT + b) * (OT * TX) + o * TX + tx] = acc[b][o];
    __syncthreads();
    for (uint32_t b = ty; b < nb; b += KS) {
#pragma unroll
        for (int o = 0; o < OT; ++o) {
            const uint32_t i = i0 + o * TX;
            if (i >= out_dim) continue;
            float v = red[b * (OT * TX) + o * TX + tx];
#pragma unroll
            for (int y = 1; y < KS; ++y) v += red[(y * BT + b) * (OT * TX) + o * TX + tx];
            out[size_t(b0 + b) * out_dim + i] = bias[i] + v;
        }
    }
}

// The same operator at decode batches (batch <= 4 per block): the whole activation rows stay in shared memory, thread
// (tx, ty) owns output i = block base + tx and every KS-th word of each group, and scale and zero point are applied once
// per group instead of once per weight:
//     sum_k x_k (q_k - zp) s  =  s (sum_k x_k q_k  -  zp sum_k x_k),
// with the activation sums of a thread's words of a group computed once per block. Per weight that leaves the nibble
// extraction, one exact subtraction and one FMA per batch row (the kernel above spends thirteen instructions per weight at
// batch 1). Same values as the operator's definition up to f32 summation order; exact whenever every partial sum is.
// grid (ceil(N / 32), ceil(B / BT)), block 32 x KS; needs (group / 8) % KS == 0.
template <int KS, int BT, int WPT>
__global__ void __launch_bounds__(32 * KS) affine_grouped_decode_kernel(const float* __restrict__ x, const uint32_t* __restrict__ w,
                                                                        const float* __restrict__ scale, const uint32_t* __restrict__ zp,
                                                                        const float* __restrict__ bias, float* __restrict__ out,
                                                                        uint32_t in_dim, uint32_t out_dim, uint32_t group, uint32_t batch) {
    extern __shared__ __align__(16) float dsm[];
    const uint32_t groups = in_dim / group, wpg = group / 8;  // words per group; WPT = wpg / KS of them are this thread's
    constexpr uint32_t wpt = WPT;
    float* xs = dsm;                                  // [BT][in_dim]
    float* xsum = dsm + size_t(BT) * in_dim;          // [BT][groups][KS]: sum of x under the words (g, j * KS + ty)
    float* red = xsum + size_t(BT) * groups * KS;     // [KS][BT][32]
    const uint32_t tx = threadIdx.x, ty = threadIdx.y, tid = ty * 32 + tx;
    const uint32_t i = blockIdx.x * 32 + tx, ic = min(i, out_dim - 1);
    const uint32_t b0 = blockIdx.y * BT, nb = min(uint32_t(BT), batch - b0);
    for (uint32_t e = tid; e < BT * (in_dim / 4); e += 32 * KS) {
        const uint32_t b = e / (in_dim / 4), k = (e % (in_dim / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < nb) v = __ldg(reinterpret_cast<const float4*>(x + size_t(b0 + b) * in_dim + k));
        *reinterpret_cast<float4*>(xs + size_t(b) * in_dim + k) = v;
    }
    __syncthreads();
    for (uint32_t e = tid; e < BT * groups * KS; e += 32 * KS) {
        const uint32_t b = e / (groups * KS), g = (e / KS) % groups, y = e % KS;
        float sum = 0.f;
        for (uint32_t j = 0; j < wpt; ++j) {
            const float* px = xs + size_t(b) * in_dim + (size_t(g) * wpg + j * KS + y) * 8;
#pragma unroll
            for (int n = 0; n < 8; ++n) sum += px[n];
        }
        xsum[e] = sum;
    }
    __syncthreads();
    float acc[BT];
#pragma unroll
    for (int b = 0; b < BT; ++b) acc[b] = 0.f;
    constexpr int GB = 4;  // groups whose words, scales and zero points are loaded together: GB * WPT words in flight per thread
    for (uint32_t g0 = 0; g0 < groups; g0 += GB) {
        uint32_t words[GB][WPT];
        float sc[GB], z[GB];
#pragma unroll
        for (int gg = 0; gg < GB; ++gg) {
            const uint32_t g = min(g0 + gg, groups - 1);  // past the end: reloaded, not used
#pragma unroll
            for (int j = 0; j < WPT; ++j) words[gg][j] = __ldg(w + size_t(g * wpg + j * KS + ty) * out_dim + ic);
            sc[gg] = __ldg(scale + size_t(g) * out_dim + ic);
            z[gg] = float(__ldg(zp + size_t(g) * out_dim + ic));
        }
#pragma unroll
        for (int gg = 0; gg < GB; ++gg) {
            const uint32_t g = g0 + gg;
            if (g >= groups) break;
            float part[BT];
#pragma unroll
            for (int b = 0; b < BT; ++b) part[b] = 0.f;
#pragma unroll
            for (int j = 0; j < WPT; ++j) {
                const uint32_t kw = g * wpg + j * KS + ty;
                const uint32_t word = words[gg][j];
                const uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu;  // nibbles 0,2,4,6 / 1,3,5,7
                float q[8];
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    // f32(nibble) without the conversion unit: 0x4B0000nn is 2^23 + nn, and the subtraction is exact
                    q[2 * n] = __uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7540 + n)) - 8388608.0f;
                    q[2 * n + 1] = __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7540 + n)) - 8388608.0f;
                }
#pragma unroll
                for (int b = 0; b < BT; ++b) {
                    const float4 xa = *reinterpret_cast<const float4*>(xs + size_t(b) * in_dim + size_t(kw) * 8);
                    const float4 xb = *reinterpret_cast<const float4*>(xs + size_t(b) * in_dim + size_t(kw) * 8 + 4);
                    float a = part[b];
                    a = fmaf(xa.x, q[0], a); a = fmaf(xa.y, q[1], a); a = fmaf(xa.z, q[2], a); a = fmaf(xa.w, q[3], a);
                    a = fmaf(xb.x, q[4], a); a = fmaf(xb.y, q[5], a); a = fmaf(xb.z, q[6], a); a = fmaf(xb.w, q[7], a);
                    part[b] = a;
                }
            }
#pragma unroll
            for (int b = 0; b < BT; ++b)
                acc[b] = fmaf(sc[gg], fmaf(-z[gg], xsum[(size_t(b) * groups + g) * KS + ty], part[b]), acc[b]);
        }
    }
    // fold the k slices in slice order (deterministic)
#pragma unroll
    for (int b = 0; b < BT; ++b) red[(ty * BT + b) * 32 + tx] = acc[b];
    __syncthreads();
    for (uint32_t b = ty; b < nb; b += KS) {
        if (i >= out_dim) continue;
        float v = red[b * 32 + tx];
        for (uint32_t y = 1; y < KS; ++y) v += red[(y * BT + b) * 32 + tx];
        out[size_t(b0 + b) * out_dim + i] = bias[i] + v;
    }
}

// one warp per row, 8 rows per block; grid (ceil(rows / 8), ceil(batch / MV_BT))
__global__ void __launch_bounds__(256) i4_matvec_fast_kernel(const uint32_t* __restrict__ w, const float* __restrict__ x,
                                                             const float* __restrict__ scales, float* __restrict__ out,
                                                             uint32_t batch, uint32_t rows, uint32_t cols) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const uint32_t b0 = blockIdx.y * MV_BT;
    const uint32_t nb = min(uint32_t(MV_BT), batch - b0);
    if (row >= rows) return;
    const uint32_t wpr = (cols + 7) / 8;
    const uint32_t* wr = w + size_t(row) * wpr;
    float acc[MV_BT];
#pragma unroll
    for (int b = 0; b < MV_BT; ++b) acc[b] = 0.0f;
    for (uint32_t wi = lane; wi < wpr; wi += 32) {
        const uint32_t word = wr[wi];
        const uint32_t c0 = wi * 8;
        float wv[8];
#pragma unroll
        for (int n = 0; n < 8; ++n) wv[n] = float(int32_t(word << (28 - 4 * n)) >> 28);  // signed nibble
        if (c0 + 8 <= cols && (cols & 3u) == 0) {
#pragma unroll
            for (int b = 0; b < MV_BT; ++b) {
                if (uint32_t(b) < nb) {
                    const float4 xa = __ldg(reinterpret_cast<const float4*>(x + size_t(b0 + b) * cols + c0));
                    const float4 xb = __ldg(reinterpret_cast<const float4*>(x + size_t(b0 + b) * cols + c0 + 4));
                    float a = acc[b];
                    a = __fmaf_rn(wv[0], xa.x, a);
                    a = __fmaf_rn(wv[1], xa.y, a);
                    a = __fmaf_rn(wv[2], xa.z, a);
                    a = __fmaf_rn(wv[3], xa.w, a);
                    a = __fmaf_rn(wv[4], xb.x, a);
                    a = __fmaf_rn(wv[5], xb.y, a);
                    a = __fmaf_rn(wv[6], xb.z, a);
                    a = __fmaf_rn(wv[7], xb.w, a);
                    acc[b] = a;
                }
            }
        } else {  // ragged tail of a row (or rows that are not 16-byte aligned)
            for (uint32_t b = 0; b < nb; ++b)
                for (uint32_t n = 0; n < 8 && c0 + n < cols; ++n)
                    acc[b] = __fmaf_rn(wv[n], x[size_t(b0 + b) * cols + c0 + n], acc[b]);
        }
    }
    const float sc = scales[row];
#pragma unroll
    for (int b = 0; b < MV_BT; ++b) {
        float v = acc[b];
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && uint32_t(b) < nb) out[size_t(b0 + b) * rows + row] = v * sc;
    }
}

}  // namespace

// shapes the fast kernels take; everything else stays on the reference-order kernels
bool affine_grouped_fast_supported(uint32_t in_dim, uint32_t out_dim, uint32_t group, uint32_t batch) {
    return in_dim % 8 == 0 && group % 8 == 0 && in_dim % group == 0 && uint64_t(in_dim) * out_dim * batch >= (1ull << 24);
}
bool i4_matvec_fast_supported(uint32_t batch, uint32_t rows, uint32_t cols) {
    return uint64_t(batch) * rows * cols >= (1ull << 22);
}

namespace {
template <int TX, int OT, int KS, int BT, int KCHUNK>
cudaError_t launch_affine_cfg(const float* x, const uint32_t* w, const float* scale, const uint32_t* zp, const float* b, float* out,
                              uint32_t in_dim, uint32_t out_dim, uint32_t group, uint32_t batch, cudaStream_t s) {
    const int shift = (group & (group - 1)) == 0 ? __builtin_ctz(group) : -1;
    const dim3 grid((out_dim + TX * OT - 1) / (TX * OT), (batch + BT - 1) / BT);
    if (grid.y > 65535u) return cudaErrorInvalidValue;
    affine_grouped_fast_kernel<TX, OT, KS, BT, KCHUNK><<<grid, dim3(TX, KS), 0, s>>>(x, w, scale, zp, b, out, in_dim, out_dim, group, shift, batch);
    return cudaGetLastError();
}
}  // namespace

cudaError_t launch_affine_grouped_fast(const float* x, const uint32_t* w, const float* scale, const uint32_t* zp,
                                       const float* b, float* out, uint32_t in_dim, uint32_t out_dim, uint32_t group,
                                       uint32_t batch, int sm_count, cudaStream_t s) {
    // decode batches: whole activation rows in shared memory, scale and zero point applied per group
    constexpr int DKS = 8;
    if (batch <= 4 && (group == 64 || group == 128) && in_dim <= 8192) {
        const int dbt = batch == 1 ? 1 : batch == 2 ? 2 : 4;
        const size_t smem = (size_t(dbt) * in_dim + size_t(dbt) * (in_dim / group) * DKS + size_t(DKS) * dbt * 32) * sizeof(float);
        const dim3 grid((out_dim + 31) / 32, 1), block(32, DKS);
        using Kernel = void (*)(const float*, const uint32_t*, const float*, const uint32_t*, const float*, float*, uint32_t, uint32_t,
                                uint32_t, uint32_t);
        static const Kernel kernels[2][3] = {
            {affine_grouped_decode_kernel<DKS, 1, 1>, affine_grouped_decode_kernel<DKS, 2, 1>, affine_grouped_decode_kernel<DKS, 4, 1>},
            {affine_grouped_decode_kernel<DKS, 1, 2>, affine_grouped_decode_kernel<DKS, 2, 2>, affine_grouped_decode_kernel<DKS, 4, 2>}};
        static std::atomic<uint64_t> configured{0};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const uint64_t bit = 1ull << (dev & 63);
        if (!(configured.load(std::memory_order_acquire) & bit)) {
            const int max_smem = int((size_t(4) * 8192 + size_t(4) * (8192 / 64) * DKS + size_t(DKS) * 4 * 32) * sizeof(float));
            for (int v = 0; v < 6 && e == cudaSuccess; ++v)
                e = cudaFuncSetAttribute((const void*)kernels[v / 3][v % 3], cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
            if (e != cudaSuccess) return e;
            configured.fetch_or(bit, std::memory_order_release);
        }
        kernels[group == 128 ? 1 : 0][dbt == 1 ? 0 : dbt == 2 ? 1 : 2]<<<grid, block, smem, s>>>(x, w, scale, zp, b, out, in_dim, out_dim,
                                                                                             group, batch);
        return cudaGetLastError();
    }
    // batch rows per block: every row beyond the batch is wasted arithmetic, every row within it reuses the dequantised weight
    const int bt = batch >= 12 ? 16 : batch >= 3 ? 8 : 2;
    // 128 outputs per block (two per thread) when that still gives every SM a block, else 32 outputs and a deeper k split
    const bool wide = uint64_t((out_dim + 127) / 128) * ((batch + bt - 1) / bt) >= uint64_t(sm_count);
#define VYB_AFFINE(TX, OT, KS, BT, KC) \
    launch_affine_cfg<TX, OT, KS, BT, KC>(x, w, scale, zp, b, out, in_dim, out_dim, group, batch, s)
    if (bt == 2) return VYB_AFFINE(32, 1, 8, 2, 2048);  // 32 words (128 B) per thread and chunk in flight, twice over
    if (wide) return bt == 16 ? VYB_AFFINE(64, 2, 4, 16, 256) : VYB_AFFINE(64, 2, 4, 8, 512);
    return bt == 16 ? VYB_AFFINE(32, 1, 8, 16, 256) : VYB_AFFINE(32, 1, 8, 8, 512);
#undef VYB_AFFINE
}

cudaError_t launch_i4_matvec_fast(const uint32_t* w, const float* x, const float* scales, float* out, uint32_t batch,
                                  uint32_t rows, uint32_t cols, cudaStream_t s) {
    i4_matvec_fast_kernel<<<dim3((rows + 7) / 8, (batch + MV_BT - 1) / MV_BT), 256, 0, s>>>(w, x, scales, out, batch, rows, cols);
    return cudaGetLastError();
}


// ---- GGML K-quant linear at size (vyre-libs/src/nn/quant/ggml.rs:217-333) ------------------------------------------------
// The weight stream is k-major with neighbouring outputs in neighbouring nibbles (2-bit fields for Q2_K), so a thread owns
// FOUR neighbouring packed word COLUMNS (one 16-byte load per k row: 32 outputs for Q4_K, 64 for Q2_K) and a warp reads 512
// contiguous bytes of one k row. The k range is cut into up to K_QUANT_K_CHUNKS chunks across blockIdx.y so that decode
// shapes fill the GPU and every thread has eight independent 16-byte loads in flight (the loop is latency-bound
// otherwise); inside a block eight k slices are folded through shared memory in slice order, the chunk's partial row goes
// to scratch, and a second launch adds the chunks in chunk order and the bias (deterministic).
// out[i] = b[i] + sum_k x[k] * (q * scale + min) with scale and minimum applied per word (x * scale once, x * min once):
// the reference's map in another summation order.
template <int BITS, int KS>
__global__ void __launch_bounds__(32 * KS) k_quant_linear_fast_kernel(const float* __restrict__ x, const uint32_t* __restrict__ packed,
                                                                      const float* __restrict__ scales, const float* __restrict__ mins,
                                                                      float* __restrict__ partial, uint32_t in_dim, uint32_t out_dim,
                                                                      uint32_t k_per_chunk) {
    constexpr int VPW = 32 / BITS;                  // outputs per packed word
    constexpr int OPT = 4 * VPW;                    // outputs per thread
    constexpr uint32_t BLOCK = BITS == 4 ? 32 : 16; // weights per scale / min
    extern __shared__ float red[];                  // [KS][32][OPT + 1]: a thread's row padded by one word, no bank conflicts
    constexpr uint32_t PITCH = 32 * (OPT + 1);
    const uint32_t tx = threadIdx.x, ky = threadIdx.y;
    const uint32_t quads_per_row = out_dim / OPT;
    const uint32_t quad = blockIdx.x * 32 + tx;
    const uint32_t k_begin = blockIdx.y * k_per_chunk, k_end = min(in_dim, k_begin + k_per_chunk);
    float acc[OPT];
#pragma unroll
    for (int j = 0; j < OPT; ++j) acc[j] = 0.f;
    if (quad < quads_per_row) {
        const uint32_t i0 = quad * OPT;
        const uint4* wp = reinterpret_cast<const uint4*>(packed);
#pragma unroll 8
        for (uint32_t k = k_begin + ky; k < k_end; k += KS) {
            const uint4 w4 = __ldg(wp + size_t(k) * quads_per_row + quad);
            const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
            const float xk = __ldg(x + k);
            const size_t lin = size_t(k) * out_dim + i0;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t blk = uint32_t((lin + w * VPW) / BLOCK);
                const float xs = xk * __ldg(scales + blk), xm = xk * __ldg(mins + blk);
#pragma unroll
                for (int j = 0; j < VPW; ++j) {
                    // the field as an f32 without an integer conversion: 2^23 + q has q in its low mantissa bits
                    const float q = __uint_as_float(0x4B000000u | ((words[w] >> (j * BITS)) & ((1u << BITS) - 1u))) - 8388608.0f;
                    acc[w * VPW + j] = fmaf(q, xs, acc[w * VPW + j] + xm);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < OPT; ++j) red[ky * PITCH + tx * (OPT + 1) + j] = acc[j];
    __syncthreads();
    for (uint32_t o = ky * 32 + tx; o < 32 * OPT; o += 32 * KS) {
        const uint32_t i = blockIdx.x * 32 * OPT + o;
        if (i >= out_dim) continue;
        float sum = 0.f;
#pragma unroll
        for (int s = 0; s < KS; ++s) sum += red[s * PITCH + (o / OPT) * (OPT + 1) + o % OPT];
        partial[size_t(blockIdx.y) * out_dim + i] = sum;
    }
}

__global__ void k_quant_fold_kernel(const float* __restrict__ partial, const float* __restrict__ b, float* __restrict__ out,
                                    uint32_t out_dim, uint32_t chunks) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= out_dim) return;
    float sum = 0.f;
#pragma unroll 16
    for (uint32_t c = 0; c < chunks; ++c) sum += __ldg(partial + size_t(c) * out_dim + i);
    out[i] = sum + b[i];
}

bool k_quant_linear_fast_supported(uint32_t in_dim, uint32_t out_dim, uint32_t bits) {
    return (bits == 4 || bits == 2) && in_dim >= 1 && out_dim >= 1 && out_dim % (4 * (32 / bits)) == 0;
}

size_t k_quant_linear_fast_scratch_bytes(uint32_t out_dim) { return size_t(K_QUANT_K_CHUNKS) * out_dim * 4; }

cudaError_t launch_k_quant_linear_fast(const float* x, const uint32_t* packed, const float* scales, const float* mins,
                                       const float* b, float* out, float* partial, uint32_t in_dim, uint32_t out_dim,
                                       uint32_t bits, int sm_count, cudaStream_t s) {
    constexpr int KS = 8;
    const uint32_t opt = 4 * (32 / bits);
    const uint32_t xblocks = (out_dim / opt + 31) / 32;
    // about two blocks per SM, 64 k rows per chunk at least (eight loads in flight per thread)
    uint32_t chunks = (2u * uint32_t(sm_count) + xblocks - 1) / xblocks;
    chunks = chunks > K_QUANT_K_CHUNKS ? K_QUANT_K_CHUNKS : chunks;
    const uint32_t by_rows = (in_dim + 63) / 64;
    chunks = chunks > by_rows ? by_rows : chunks;
    const uint32_t k_per_chunk = (in_dim + chunks - 1) / chunks;
    chunks = (in_dim + k_per_chunk - 1) / k_per_chunk;
    const dim3 grid(xblocks, chunks), block(32, KS);
    const size_t smem = size_t(KS) * 32 * (opt + 1) * 4;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t de = cudaGetDevice(&dev);
    if (de != cudaSuccess) return de;
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(k_quant_linear_fast_kernel<2, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             int(size_t(KS) * 32 * 65 * 4));
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit, std::memory_order_release);
    }
    if (bits == 4)
        k_quant_linear_fast_kernel<4, KS><<<grid, block, smem, s>>>(x, packed, scales, mins, partial, in_dim, out_dim, k_per_chunk);
    else
        k_quant_linear_fast_kernel<2, KS><<<grid, block, smem, s>>>(x, packed, scales, mins, partial, in_dim, out_dim, k_per_chunk);
    k_quant_fold_kernel<<<(out_dim + 255) / 256, 256, 0, s>>>(partial, b, out, out_dim, chunks);
    return cudaGetLastError();
}

}  // namespace vybk
