// int8 x int8 -> int32 GEMM on CTA pairs (tcgen05 cta_group::2, sm_100a).
//
//   out[m, n] = sum_k a[m, k] * w[n, k]        a int8 [M, K], w int8 [N, K] (both K-major), out int32 [M, N]
//
// Same arithmetic as the single-CTA kernel (bit-exact; the two's-complement reading of the reference's wrapping-u32
// Matmul, vyre-libs/src/math/linalg/matmul.rs:17-60). Two CTAs of a cluster own a 256 x 256 output tile: each loads
// its own 128 activation rows and HALF of the tile's weight rows (128 x 128-byte boxes, 128-byte swizzle, 6 stages of
// 32 KB per CTA), both counted on the leader's mbarrier; the leader issues tcgen05.mma.cta_group::2.kind::i8 (M = 256,
// N = 256, K = 32); every CTA drains its 128 accumulator rows from its own TMEM. Per SM this halves the weight bytes
// read from L2 and the operand bytes the tensor core reads from shared memory compared with one CTA per 128 x 256 tile.
// Roles by SM sub-partition: warp 0 TMA, warp 4 MMA + TMEM owner, warps 8, 1, 2, 3 epilogue. Two accumulators overlap
// the epilogue with the next tile. Every wait is clock-bounded and raises a status word. No multicast.
#include <atomic>

#include "kernels.h"
#include "tcgen05_common.cuh"

namespace vybk {
namespace {

using namespace tc;

constexpr int BM = 128;   // rows per CTA (256 per pair)
constexpr int BN = 256;   // accumulator columns per pair tile (128 weight rows per CTA)
constexpr int BK = 128;   // bytes = int8 elements per stage row
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK, B_BYTES = (BN / 2) * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMA_WARP = 0, MMA_WARP = 4;
constexpr int NUM_WARPS = 9;
constexpr int THREADS = NUM_WARPS * 32;
constexpr int TMEM_COLS = 512;
constexpr int GSTAGE_PITCH = 36;                       // 32-bit words per staged row: 16-byte aligned, conflict-free v4 stores
constexpr int GSTAGE_BYTES = 4 * 32 * GSTAGE_PITCH * 4;  // one 32 x 32 block per epilogue warp (the gathering form)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + GSTAGE_BYTES;

struct Bars {
    unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    unsigned int abort_flag;
};

__device__ __forceinline__ bool is_epilogue_warp(int w) { return w == 8 || (w >= 1 && w <= 3); }

__global__ void __launch_bounds__(THREADS, 1)
int8_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      int32_t* __restrict__ out, uint32_t M, uint32_t N, uint32_t K, uint32_t* status,
                      const GemmGatherOut go) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Bars* bars = reinterpret_cast<Bars*>(tiles + STAGES * STAGE_BYTES);
    uint32_t* gstage = reinterpret_cast<uint32_t*>(tiles + STAGES * STAGE_BYTES + 256);  // behind the barriers
    volatile unsigned int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + BN - 1) / BN;
    const uint32_t total_tiles = m_tiles * n_tiles, k_blocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);   // leader: one expect_tx arrival, bytes from both CTAs
            mbar_init(smem_u32(&bars->empty[s]), 1);  // one tcgen05.commit per CTA
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars->acc_full[a]), 1);
            mbar_init(smem_u32(&bars->acc_empty[a]), 8);  // leader: 4 epilogue warps of each CTA
        }
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_w);
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(smem_u32(&bars->tmem_base), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == TMA_WARP) {
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t tile = pair; tile < total_tiles && ok; tile += pairs) {
            const int m0 = int((tile % m_tiles) * 2 * BM + rank * BM);
            const int n0 = int((tile / m_tiles) * BN + rank * (BN / 2));
            for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it) {
                const uint32_t s = it % STAGES;
                if (it >= STAGES) ok = mbar_wait(smem_u32(&bars->empty[s]), ((it / STAGES) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t leader_bar = mapa(smem_u32(&bars->full[s]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bars->full[s]), 2 * STAGE_BYTES);
                    uint8_t* st = tiles + size_t(s) * STAGE_BYTES;
                    tma_load_2d_pair(smem_u32(st), &map_a, int(kb * BK), m0, leader_bar);
                    tma_load_2d_pair(smem_u32(st + A_BYTES), &map_w, int(kb * BK), n0, leader_bar);
                }
                __syncwarp();
            }
        }
    } else if (warp == MMA_WARP) {
        if (rank == 0) {
            constexpr uint32_t idesc = idesc_s8_s32(2 * BM, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (uint32_t tile = pair; tile < total_tiles && ok; tile += pairs, ++local) {
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
                            mma_i8_pair(d_tmem, smem_desc_advance(da, k * UMMA_K), smem_desc_advance(db, k * UMMA_K), idesc,
                                        (kb | uint32_t(k)) != 0);
                        const uint32_t em = smem_u32(&bars->empty[s]);
                        tc_commit_pair(em);
                        tc_commit_pair(mapa(em, 1));
                    }
                    __syncwarp();
                }
                if (ok && lane == 0) {
                    const uint32_t af = smem_u32(&bars->acc_full[acc]);
                    tc_commit_pair(af);
                    tc_commit_pair(mapa(af, 1));
                }
                __syncwarp();
            }
        }
    } else if (is_epilogue_warp(warp)) {
        const uint32_t quad = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (uint32_t tile = pair; tile < total_tiles && ok; tile += pairs, ++local) {
            const uint32_t acc = local & 1;
            const uint32_t m0 = (tile % m_tiles) * 2 * BM + rank * BM, n0 = (tile / m_tiles) * BN;
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
                    if (go.count == 0) {
                        int32_t* dst = out + size_t(row) * N + col0;
                        if (col0 + 32 <= N && (N & 3u) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4*>(dst)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) dst[j] = int32_t(r[j]);
                        }
                    }
                }
                if (go.count != 0) {
                    // The gathering form: this rank's columns go straight into every rank's full output (peer stores over
                    // NVLink for the others) while the MMA warp is already on the next tile. A lane holds one ROW of the
                    // 32 x 32 block; stored like that, every 16-byte store of a warp would land in a different row. The
                    // block goes through shared memory instead, and eight lanes store 128 contiguous bytes of a row.
                    uint32_t* stage = gstage + quad * (32 * GSTAGE_PITCH);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<uint4*>(stage + lane * GSTAGE_PITCH + 4 * j) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    __syncwarp();
                    const uint32_t sub = lane >> 3, chunk = lane & 7;  // four rows per store instruction
                    const uint32_t col = col0 + chunk * 4;
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) {
                        const uint32_t brow = rr * 4 + sub, grow = m0 + quad * 32 + brow;
                        const uint4 v = *reinterpret_cast<const uint4*>(stage + brow * GSTAGE_PITCH + chunk * 4);
                        if (grow < M && col < N) {  // N is a multiple of 4: a 16-byte piece is inside or outside
                            const size_t at = size_t(grow) * go.pitch + go.col_off + col;
                            for (uint32_t d = 0; d < go.count; ++d) *reinterpret_cast<uint4*>(reinterpret_cast<int32_t*>(go.dst[d]) + at) = v;
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&bars->acc_empty[acc]), 0));
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer may still be reading this CTA's shared memory / TMEM through the pair MMA until here
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && bars->abort_flag != 0 && status) atomicOr(status, 32u);
}

}  // namespace

bool int8_gemm_pair_supported(uint32_t m, uint32_t n, uint32_t k) {
    return m > 128 && n >= 1 && k >= 16 && k % 16 == 0 && k <= 132096;
}

namespace {
cudaError_t launch_pair(const int8_t* a, const int8_t* w, int32_t* out, uint32_t m, uint32_t n, uint32_t k, int sm_count,
                        cudaStream_t stream, uint32_t* status, const GemmGatherOut& go) {
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load() & bit)) {
        e = cudaFuncSetAttribute(int8_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit);
    }
    const uint32_t pairs_avail = uint32_t(sm_count) / 2;
    if (pairs_avail == 0) return cudaErrorInvalidConfiguration;
    CUtensorMap ma, mw;
    if (!encode_tensor_map_2d(&ma, a, m, k, 1, BM, BK, true) || !encode_tensor_map_2d(&mw, w, n, k, 1, BN / 2, BK, true))
        return cudaErrorInvalidValue;
    const uint32_t tiles = ((m + 2 * BM - 1) / (2 * BM)) * ((n + BN - 1) / BN);
    const uint32_t pairs = tiles < pairs_avail ? tiles : pairs_avail;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, int8_gemm_pair_kernel, ma, mw, out, m, n, k, status, go);
    return e != cudaSuccess ? e : cudaGetLastError();
}
}  // namespace

cudaError_t launch_int8_gemm_pair(const int8_t* a, const int8_t* w, int32_t* out, uint32_t m, uint32_t n, uint32_t k,
                                  int sm_count, cudaStream_t stream, uint32_t* status) {
    return launch_pair(a, w, out, m, n, k, sm_count, stream, status, GemmGatherOut{});
}

cudaError_t launch_int8_gemm_pair_gather(const int8_t* a, const int8_t* w, const GemmGatherOut& go, uint32_t m, uint32_t n,
                                         uint32_t k, int sm_count, cudaStream_t stream, uint32_t* status) {
    if (go.count < 1 || go.count > 8 || (go.pitch | go.col_off | n) % 4 || !int8_gemm_pair_supported(m, n, k))
        return cudaErrorInvalidValue;
    for (uint32_t d = 0; d < go.count; ++d)
        if (!go.dst[d] || (go.dst[d] & 15)) return cudaErrorInvalidValue;
    return launch_pair(a, w, nullptr, m, n, k, sm_count, stream, status, go);
}

}  // namespace vybk
