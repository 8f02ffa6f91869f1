// Prefill GEMM for group-quantized int4 weights on the 5th-generation tensor cores (tcgen05, sm_100a):
//
//   y[m, n] = bf16|f32( sum_k x[m, k] * bf16((q[n, k] - 8) * s[n, k / group]) )      f32 accumulate in TMEM
//
// With hundreds of activation rows the op is a dense contraction, so it runs on the tensor cores; the weights
// stay packed in HBM and L2 and are dequantised to bf16 tiles on the fly, inside the kernel, straight into
// the swizzled shared-memory layout the MMA reads.
//
// One persistent CTA per SM walks 128 (rows of x) x 256 (rows of W) output tiles, M fastest. Per 64-k stage:
//   * warp 0 issues two TMA tensor loads: the bf16 activation box (128 x 64, 128-byte swizzle) and the raw
//     packed-weight box (256 rows x 32 bytes);
//   * 16 dequant warps (two threads per weight row) read their 16 raw bytes, turn each nibble pair into bf16 with
//     the (w & 0x000F000F) | 0x43004300 magic (= 128+q exactly), subtract 136 and multiply by the group scale
//     with packed bf16 arithmetic (one rounding: bf16((q-8)*s)), and store 4 x 16 B into the 128-byte-swizzled
//     K-major tile (chunk j of row r goes to chunk j ^ (r & 7), which is also bank-conflict free), then fence the
//     generic-proxy writes towards the async proxy and arrive on the stage barrier;
//   * one thread of warp 1 issues 4 x tcgen05.mma.kind::f16 (M=128, N=256, K=16) per stage from shared-memory
//     descriptors; tcgen05.commit releases the stage;
//   * 4 epilogue warps drain the 128 x 256 f32 accumulator from TMEM (tcgen05.ld) and store bf16 (or f32) rows.
// Two accumulators (512 TMEM columns) overlap the epilogue of tile i with the main loop of tile i+1.
// Every mbarrier wait is bounded; a wait that runs out raises a status word, the CTA drains and frees its TMEM.
//
// Replaces, for large batches, the generated scalar kernel of
// vyre-libs/src/nn/linear/inner/linear_4bit.rs:399-775; the tile layout is the row-major primitive layout of
// vyre-primitives/src/math/quantized/programs.rs:181.
#include <cuda_bf16.h>

#include <atomic>

#include "kernels.h"
#include "tcgen05_common.cuh"

namespace vybk {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64;  // BK in bf16 elements (128 bytes per row)
constexpr int UMMA_K = 16;
// Three independent rings: the packed weights are prefetched deepest (they are small and come from HBM/L2), the
// activation boxes next, and the dequantised tiles (the large ones) only need to cover dequant + MMA latency.
constexpr int A_STAGES = 4, RAW_STAGES = 8, B_STAGES = 3;
constexpr int RAW_AHEAD = 4;              // raw loads run this many stages ahead of the activation loads
constexpr int A_BYTES = BM * BK * 2;      // 16 KB activations
constexpr int B_BYTES = BN * BK * 2;      // 32 KB dequantised weights
constexpr int RAW_BYTES = BN * (BK / 2);  // 8 KB packed weights
constexpr int B_RING = 0, A_RING = B_STAGES * B_BYTES, RAW_RING = A_RING + A_STAGES * A_BYTES;
constexpr int RING_BYTES = RAW_RING + RAW_STAGES * RAW_BYTES;
constexpr int DEQ_WARPS = 16;                 // two threads per weight row (32 k each)
constexpr int THREADS = (6 + DEQ_WARPS) * 32;  // TMA, MMA, 4 epilogue, 16 dequant
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = RING_BYTES + 1024 + 512;

struct Bars {
    unsigned long long a_full[A_STAGES], a_empty[A_STAGES], raw_full[RAW_STAGES], raw_empty[RAW_STAGES];
    unsigned long long b_full[B_STAGES], b_empty[B_STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    unsigned int abort_flag;
};

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

template <bool OUT_F32>
__global__ void __launch_bounds__(THREADS, 1)
int4_prefill_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const uint16_t* __restrict__ scales, void* __restrict__ y, uint32_t M, uint32_t N, uint32_t K,
                    uint32_t group, uint32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Bars* bars = reinterpret_cast<Bars*>(tiles + RING_BYTES);
    volatile unsigned int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const uint32_t total_tiles = m_tiles * n_tiles, k_blocks = (K + BK - 1) / BK;
    const uint32_t groups = K / group;

    if (threadIdx.x == 0) {
        for (int s = 0; s < A_STAGES; ++s) {
            mbar_init(smem_u32(&bars->a_full[s]), 1);
            mbar_init(smem_u32(&bars->a_empty[s]), 1);
        }
        for (int s = 0; s < RAW_STAGES; ++s) {
            mbar_init(smem_u32(&bars->raw_full[s]), 1);
            mbar_init(smem_u32(&bars->raw_empty[s]), DEQ_WARPS);
        }
        for (int s = 0; s < B_STAGES; ++s) {
            mbar_init(smem_u32(&bars->b_full[s]), DEQ_WARPS);
            mbar_init(smem_u32(&bars->b_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars->acc_full[a]), 1);
            mbar_init(smem_u32(&bars->acc_empty[a]), 4);
        }
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&bars->tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
        // ------------------------------------ TMA producer ------------------------------------
        // two cursors over the same (tile, k-block) sequence: the raw-weight cursor leads the activation cursor
        uint32_t a_it = 0, r_it = 0, r_tile = blockIdx.x, r_kb = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int m0 = int(tile % m_tiles) * BM;
            for (uint32_t kb = 0; kb < k_blocks && ok; ++kb, ++a_it) {
                while (ok && r_tile < total_tiles && r_it <= a_it + RAW_AHEAD) {
                    const uint32_t rs = r_it % RAW_STAGES;
                    if (r_it >= RAW_STAGES)
                        ok = mbar_wait(smem_u32(&bars->raw_empty[rs]), ((r_it / RAW_STAGES) - 1) & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    if (lane == 0) {
                        const uint32_t bar = smem_u32(&bars->raw_full[rs]);
                        mbar_arrive_expect_tx(bar, RAW_BYTES);
                        tma_load_2d(smem_u32(tiles + RAW_RING + rs * RAW_BYTES), &map_w, int(r_kb * (BK / 2)),
                                    int(r_tile / m_tiles) * BN, bar);
                    }
                    __syncwarp();
                    ++r_it;
                    if (++r_kb == k_blocks) {
                        r_kb = 0;
                        r_tile += gridDim.x;
                    }
                }
                if (!ok) break;
                const uint32_t as = a_it % A_STAGES;
                if (a_it >= A_STAGES) ok = mbar_wait(smem_u32(&bars->a_empty[as]), ((a_it / A_STAGES) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t bar = smem_u32(&bars->a_full[as]);
                    mbar_arrive_expect_tx(bar, A_BYTES);
                    tma_load_2d(smem_u32(tiles + A_RING + as * A_BYTES), &map_x, int(kb * BK), m0, bar);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ------------------------------------ MMA issuer ---------------------------------------
        constexpr uint32_t idesc = idesc_bf16_f32(BM, BN);
        uint32_t it = 0, local = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            const uint32_t acc = local & 1;
            if (local >= 2) ok = mbar_wait(smem_u32(&bars->acc_empty[acc]), ((local >> 1) - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it) {
                const uint32_t as = it % A_STAGES, bs = it % B_STAGES;
                ok = mbar_wait(smem_u32(&bars->a_full[as]), (it / A_STAGES) & 1, abort_flag) &&
                     mbar_wait(smem_u32(&bars->b_full[bs]), (it / B_STAGES) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint64_t da = smem_desc_sw128(smem_u32(tiles + A_RING + as * A_BYTES));
                    const uint64_t db = smem_desc_sw128(smem_u32(tiles + B_RING + bs * B_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_f16(d_tmem, smem_desc_advance(da, k * UMMA_K * 2), smem_desc_advance(db, k * UMMA_K * 2), idesc,
                                (kb | uint32_t(k)) != 0);
                    tc_commit(smem_u32(&bars->a_empty[as]));
                    tc_commit(smem_u32(&bars->b_empty[bs]));
                }
                __syncwarp();
            }
            if (ok && lane == 0) tc_commit(smem_u32(&bars->acc_full[acc]));
            __syncwarp();
        }
    } else if (warp < 6) {
        // ------------------------------------ epilogue warps ------------------------------------
        const uint32_t quad = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
            const uint32_t acc = local & 1;
            const uint32_t m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            ok = mbar_wait(smem_u32(&bars->acc_full[acc]), (local >> 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t row = m0 + quad * 32 + lane;
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + c * 32, r);
                tmem_ld_wait();
                const uint32_t col0 = n0 + c * 32;
                if (row < M && col0 < N) {
                    if constexpr (OUT_F32) {
                        float* dst = static_cast<float*>(y) + size_t(row) * N + col0;
                        if (col0 + 32 <= N && (N & 3u) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4*>(dst)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) dst[j] = __uint_as_float(r[j]);
                        }
                    } else {
                        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(y) + size_t(row) * N + col0;
                        if (col0 + 32 <= N && (N & 7u) == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                uint32_t pk[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * q]),
                                                                                   __uint_as_float(r[8 * j + 2 * q + 1]));
                                    pk[q] = *reinterpret_cast<const uint32_t*>(&h);
                                }
                                reinterpret_cast<uint4*>(dst)[j] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            }
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[acc]));
        }
    } else {
        // ------------------------------------ dequant warps ------------------------------------
        const uint32_t tid = (warp - 6) * 32 + lane;
        const uint32_t r = tid >> 1;     // weight row inside the tile
        const uint32_t half = tid & 1u;  // which 32-k half of the 64-k stage row
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const uint32_t n0 = (tile / m_tiles) * BN;
            const bool row_valid = n0 + r < N;
            const uint16_t* srow = scales + size_t(row_valid ? n0 + r : 0) * groups;
            // scales are read one group ahead: the load issued at a group change is consumed at the next one,
            // so its latency hides behind a whole group of dequantisation instead of stalling every other stage
            uint32_t cur_group = 0xFFFFFFFFu, s2 = 0;
            uint32_t s_next = row_valid ? uint32_t(srow[0]) : 0u;
            for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it) {
                const uint32_t rs = it % RAW_STAGES, bs = it % B_STAGES;
                const uint32_t g = (kb * BK) / group;
                if (g != cur_group) {
                    cur_group = g;
                    s2 = s_next | (s_next << 16);  // this group's scale in both bf16 halves
                    s_next = (row_valid && g + 1 < groups) ? uint32_t(srow[g + 1]) : 0u;
                }
                ok = mbar_wait(smem_u32(&bars->raw_full[rs]), (it / RAW_STAGES) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint4 w0 = *reinterpret_cast<const uint4*>(tiles + RAW_RING + rs * RAW_BYTES + r * (BK / 2) + half * 16);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->raw_empty[rs]));  // the packed bytes now live in registers
                const uint32_t words[4] = {w0.x, w0.y, w0.z, w0.w};
                uint4 o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t w = words[j];
                    uint32_t t0 = (w & 0x000F000Fu) | 0x43004300u;          // (k0, k4) as 128+q
                    uint32_t t1 = ((w >> 4) & 0x000F000Fu) | 0x43004300u;   // (k1, k5)
                    uint32_t t2 = ((w >> 8) & 0x000F000Fu) | 0x43004300u;   // (k2, k6)
                    uint32_t t3 = ((w >> 12) & 0x000F000Fu) | 0x43004300u;  // (k3, k7)
                    t0 = bf16x2_mul(bf16x2_sub(t0, 0x43084308u), s2);       // exact q-8, then one rounding of (q-8)*s
                    t1 = bf16x2_mul(bf16x2_sub(t1, 0x43084308u), s2);
                    t2 = bf16x2_mul(bf16x2_sub(t2, 0x43084308u), s2);
                    t3 = bf16x2_mul(bf16x2_sub(t3, 0x43084308u), s2);
                    o[j].x = __byte_perm(t0, t1, 0x5410);  // (k0, k1)
                    o[j].y = __byte_perm(t2, t3, 0x5410);  // (k2, k3)
                    o[j].z = __byte_perm(t0, t1, 0x7632);  // (k4, k5)
                    o[j].w = __byte_perm(t2, t3, 0x7632);  // (k6, k7)
                }
                // the dequantised tile slot must have been consumed by the MMAs of its previous use
                if (it >= B_STAGES) ok = mbar_wait(smem_u32(&bars->b_empty[bs]), ((it / B_STAGES) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                uint8_t* brow = tiles + B_RING + bs * B_BYTES + r * 128;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t chunk = half * 4 + uint32_t(j);
                    *reinterpret_cast<uint4*>(brow + ((chunk ^ (r & 7u)) << 4)) = o[j];
                }
                fence_proxy_async();  // make the generic-proxy stores visible to the tensor core's operand reads
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->b_full[bs]));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && bars->abort_flag != 0 && status) atomicOr(status, 8u);
}

}  // namespace

bool int4_prefill_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    // 64-k stages must not straddle a scale group; tensor-map strides need 16-byte multiples
    return m >= 1 && n >= 1 && k >= 64 && k % 64 == 0 && group >= 64 && group % 64 == 0 && k % group == 0;
}

cudaError_t launch_int4_prefill(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                uint32_t n, uint32_t k, uint32_t group, uint32_t out_f32, int sm_count,
                                cudaStream_t stream, uint32_t* status) {
    // above 128 rows the CTA-pair kernel (256-row tiles, half the dequantisation per SM) takes over
    if (int4_gemm_pair_supported(m, n, k, group) && sm_count >= 2)
        return launch_int4_gemm_pair(x_bf16, w_packed, scale_bf16, y, m, n, k, group, out_f32, 0, 1, nullptr, nullptr, n,
                                     sm_count, stream, status);
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load() & bit)) {
        e = cudaFuncSetAttribute(int4_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(int4_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit);
    }
    CUtensorMap mx, mw;
    if (!encode_tensor_map_2d(&mx, x_bf16, m, k, 2, BM, BK, true) ||
        !encode_tensor_map_2d(&mw, w_packed, n, k / 2, 1, BN, BK / 2, false))
        return cudaErrorInvalidValue;
    const uint32_t tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const uint32_t grid = tiles < uint32_t(sm_count) ? tiles : uint32_t(sm_count);
    if (out_f32)
        int4_prefill_kernel<true><<<grid, THREADS, SMEM_BYTES, stream>>>(mx, mw, static_cast<const uint16_t*>(scale_bf16),
                                                                         y, m, n, k, group, status);
    else
        int4_prefill_kernel<false><<<grid, THREADS, SMEM_BYTES, stream>>>(mx, mw, static_cast<const uint16_t*>(scale_bf16),
                                                                          y, m, n, k, group, status);
    return cudaGetLastError();
}

}  // namespace vybk
