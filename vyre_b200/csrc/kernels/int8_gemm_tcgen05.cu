// int8 x int8 -> int32 GEMM on the 5th-generation tensor cores (tcgen05, sm_100a), plus the per-token
// activation quantiser that feeds it.
//
//   out[m, n] = sum_k a[m, k] * w[n, k]        a int8 [M, K], w int8 [N, K] (both K-major), out int32 [M, N]
//
// Bit-exact integer arithmetic: the two's-complement reading of the reference's wrapping-u32 Matmul
// (vyre-libs/src/math/linalg/matmul.rs:17-60) on sign-extended bytes; K * 127^2 < 2^31 for every K this path
// accepts, so nothing wraps.
//
// One persistent CTA per SM walks 128 x 256 output tiles (M fastest, so the CTAs of a wave share one weight
// tile through L2). Roles: warp 0 issues TMA tensor loads (128-byte swizzled boxes, 128 k per stage, 4 stages
// of 48 KB); one thread of warp 1 issues tcgen05.mma.kind::i8 (M=128, N=256, K=32) with both operands read from
// shared memory through descriptors and the s32 accumulator in TMEM; warps 2-5 drain the accumulator with
// tcgen05.ld and store int32 rows. Two 256-column accumulators (all 512 TMEM columns) let the epilogue of tile
// i overlap the main loop of tile i+1. Every mbarrier wait is bounded; a wait that runs out raises a status
// word, the CTA drains, frees its TMEM and returns.
#include <atomic>

#include "kernels.h"
#include "tcgen05_common.cuh"

namespace vybk {

bool encode_tensor_map_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t elem_bytes,
                          uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static std::atomic<EncodeFn> cached{nullptr};
    EncodeFn fn = cached.load();
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return false;
        fn = reinterpret_cast<EncodeFn>(p);
        cached.store(fn);
    }
    const CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * elem_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 128;  // BK in bytes = int8 elements
constexpr int UMMA_K = 32;                   // k per tcgen05.mma for 8-bit operands
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct Bars {
    unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    unsigned int abort_flag;
};

__global__ void __launch_bounds__(THREADS, 1)
int8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, int32_t* out,
                 uint32_t M, uint32_t N, uint32_t K, uint32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Bars* bars = reinterpret_cast<Bars*>(tiles + STAGES * STAGE_BYTES);
    volatile unsigned int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const uint32_t total_tiles = m_tiles * n_tiles, k_blocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars->acc_full[a]), 1);
            mbar_init(smem_u32(&bars->acc_empty[a]), 4);
        }
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&map_a);
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
        // the whole warp walks the loop (so it reconverges for the final block barrier); lane 0 issues
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int m0 = int(tile % m_tiles) * BM, n0 = int(tile / m_tiles) * BN;
            for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it) {
                const uint32_t s = it % STAGES;
                if (it >= STAGES) ok = mbar_wait(smem_u32(&bars->empty[s]), ((it / STAGES) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t bar = smem_u32(&bars->full[s]);
                    uint8_t* st = tiles + size_t(s) * STAGE_BYTES;
                    mbar_arrive_expect_tx(bar, STAGE_BYTES);
                    tma_load_2d(smem_u32(st), &map_a, int(kb * BK), m0, bar);
                    tma_load_2d(smem_u32(st + A_BYTES), &map_w, int(kb * BK), n0, bar);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ------------------------------------ MMA issuer ---------------------------------------
        constexpr uint32_t idesc = idesc_s8_s32(BM, BN);
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
                const uint32_t s = it % STAGES;
                ok = mbar_wait(smem_u32(&bars->full[s]), (it / STAGES) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint8_t* st = tiles + size_t(s) * STAGE_BYTES;
                    const uint64_t da = smem_desc_sw128(smem_u32(st));
                    const uint64_t db = smem_desc_sw128(smem_u32(st + A_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        mma_i8(d_tmem, smem_desc_advance(da, k * UMMA_K), smem_desc_advance(db, k * UMMA_K), idesc,
                               (kb | uint32_t(k)) != 0);
                    tc_commit(smem_u32(&bars->empty[s]));  // stage reusable once these MMAs have read it
                }
                __syncwarp();
            }
            if (ok && lane == 0) tc_commit(smem_u32(&bars->acc_full[acc]));
            __syncwarp();
        }
    } else {
        // ------------------------------------ epilogue warps ------------------------------------
        const uint32_t quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
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
                    int32_t* dst = out + size_t(row) * N + col0;
                    if (col0 + 32 <= N && (N & 3u) == 0) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            reinterpret_cast<int4*>(dst)[j] = make_int4(int(r[4 * j]), int(r[4 * j + 1]), int(r[4 * j + 2]), int(r[4 * j + 3]));
                    } else {
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < N) dst[j] = int32_t(r[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->acc_empty[acc]));
        }
    }

    // teardown: everybody meets here (every loop above is bounded), then the allocating warp frees TMEM
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && bars->abort_flag != 0 && status) atomicOr(status, 4u);
}

// Per-token symmetric int8 quantisation: s_t = max|x| / 127, q = clamp(rint(x / s_t), -127, 127); one warp per row.
__global__ void __launch_bounds__(256) quantize_per_token_kernel(const uint16_t* __restrict__ x, int8_t* __restrict__ q,
                                                                float* __restrict__ scales, uint32_t M, uint32_t K) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const uint16_t* xr = x + size_t(row) * K;
    float amax = 0.0f;
    for (uint32_t k = lane; k < K; k += 32) amax = fmaxf(amax, fabsf(__uint_as_float(uint32_t(xr[k]) << 16)));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    if (lane == 0) scales[row] = s;
    for (uint32_t k = lane; k < K; k += 32) {
        const float v = __fdiv_rn(__uint_as_float(uint32_t(xr[k]) << 16), s);
        q[size_t(row) * K + k] = int8_t(fminf(127.0f, fmaxf(-127.0f, rintf(v))));
    }
}

}  // namespace

cudaError_t launch_quantize_per_token_int8(const void* x_bf16, int8_t* q, float* scales, uint32_t m, uint32_t k,
                                           cudaStream_t stream) {
    quantize_per_token_kernel<<<(m + 7) / 8, 256, 0, stream>>>(static_cast<const uint16_t*>(x_bf16), q, scales, m, k);
    return cudaGetLastError();
}

bool int8_gemm_supported(uint32_t m, uint32_t n, uint32_t k) {
    // tensor-map strides must be multiples of 16 bytes; the int32 sums must not wrap: activations are clamped to
    // +-127 but a weight may be -128, so k * 127 * 128 must stay below 2^31 (k <= 132104)
    return m >= 1 && n >= 1 && k >= 16 && k % 16 == 0 && k <= 132096;
}

cudaError_t launch_int8_gemm(const int8_t* a, const int8_t* w, int32_t* out, uint32_t m, uint32_t n, uint32_t k,
                             int sm_count, cudaStream_t stream, uint32_t* status) {
    // from two waves of 256 x 256 pair tiles on, the CTA-pair kernel takes over (below that, 128 x 256 tiles on single
    // SMs fill the machine better)
    const uint32_t pair_tiles = ((m + 255) / 256) * ((n + 255) / 256);
    if (int8_gemm_pair_supported(m, n, k) && sm_count >= 2 && pair_tiles >= 2 * uint32_t(sm_count / 2))
        return launch_int8_gemm_pair(a, w, out, m, n, k, sm_count, stream, status);
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load() & bit)) {
        e = cudaFuncSetAttribute(int8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit);
    }
    CUtensorMap ma, mw;
    if (!encode_tensor_map_2d(&ma, a, m, k, 1, BM, BK, true) || !encode_tensor_map_2d(&mw, w, n, k, 1, BN, BK, true))
        return cudaErrorInvalidValue;
    const uint32_t tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const uint32_t grid = tiles < uint32_t(sm_count) ? tiles : uint32_t(sm_count);
    int8_gemm_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(ma, mw, out, m, n, k, status);
    return cudaGetLastError();
}

}  // namespace vybk
