// int4 group-quantized GEMM on CTA pairs (tcgen05 cta_group::2, sm_100a): dense prefill, grouped (per-expert) and
// grouped with a fused SwiGLU epilogue.
//
//   plain:  y[m, n]  = bf16|f32( sum_k x[m, k] * bf16((q[e(m), n, k] - 8) * s[e(m), n, k / group]) )
//   glu:    h[m, j]  = bf16( g * (u * sigmoid(g)) ),  g = bf16(x[m,:] . W1[e(m), j, :]),  u = bf16(x[m,:] . W3[e(m), j, :])
//
// Two CTAs of a cluster (one TPC) share every MMA: the pair owns a 256-row x BN-column accumulator tile, each CTA
// holds its own 128 activation rows and HALF of the weight rows of the tile, and the leader CTA issues
// tcgen05.mma.cta_group::2 (M = 256). Compared with one CTA per 128 x 256 tile this halves, per SM, the packed
// weights that are dequantised, the bf16 tile bytes written to shared memory and the operand bytes the tensor
// core reads from it - the three things that bound the single-CTA kernel.
//
// Roles per CTA (20 warps, placed by SM sub-partition = warp id % 4): warp 0 TMA producer (activation box -> the
// LEADER's barrier with the pair form of the tensor load; packed-weight box -> a local barrier), warp 4 TMEM owner
// (+ MMA issuer in the leader); warps 8, 1, 2, 3 epilogue (tcgen05.ld -> global); the twelve warps >= 5 outside
// sub-partition 0 dequantise in three groups of four: group g takes the stages with stage % 3 == g, one weight row
// per thread, so three stages are always in flight (one group per stage could not keep up with the MMAs).
// Activation and dequantised tiles share a 6-stage ring of 64 k with one "consumed" barrier per CTA (two
// tcgen05.commit per stage); packed weights arrive 256 k at a time as 128-byte swizzled rows (2 slots) - 32-byte
// rows cost four times the TMA requests and starved the pipeline. Group scales are prefetched four stages ahead
// into registers (an L2 hit takes longer than a stage).
// In glu mode the leader dequantises the gate rows and the peer the up rows of the same 128 output columns, so the
// epilogue finds g in accumulator columns [0, BN/2) and u in [BN/2, BN) of its own TMEM.
// BN is 256 unless the problem is narrower (a multiple of 32, or 64 for glu).
//
// Remote mbarrier arrives use the default semantics: an explicit cluster-scope release made every arrive wait for
// a cluster-wide fence (~2000 cycles each, measured).
//
// Every wait is clock-bounded; on expiry the CTA raises a status word, drains and frees its TMEM. No multicast.
//
// Replaces, for large batches, the generated scalar kernel of
// vyre-libs/src/nn/linear/inner/linear_4bit.rs:399-775 and, in grouped form, the per-token expert_mlp of
// vyre-libs/src/nn/moe/expert_mlp.rs:18-150 (SwiGLU order of vyre-libs/src/nn/activation/unary.rs:79-100).
#include <cuda_bf16.h>

#include <atomic>

#include "kernels.h"
#include "tcgen05_common.cuh"

namespace vybk {
namespace {

using namespace tc;

constexpr int BM = 128;  // activation rows per CTA (256 per pair)
constexpr int BK = 64;   // bf16 elements per stage row (128 bytes)
constexpr int UMMA_K = 16;
constexpr int MAX_BN = 256;
constexpr int STAGES = 6;  // activation and dequantised tiles share one ring index and one 'consumed' barrier
constexpr int A_STAGES = STAGES, B_STAGES = STAGES, RAW_STAGES = 2, RAW_AHEAD = 1;
constexpr int RAW_KB = 4;  // k-blocks per packed-weight load: 128-byte rows, a quarter of the TMA requests of 32-byte rows
constexpr int A_BYTES = BM * BK * 2;                 // 16 KB
constexpr int B_BYTES = (MAX_BN / 2) * BK * 2;       // 16 KB: this CTA's half of the dequantised tile
constexpr int RAW_BYTES = (MAX_BN / 2) * RAW_KB * (BK / 2);  // 16 KB: 128 rows x 128 bytes (256 k), 128-byte swizzle
constexpr int B_RING = 0, A_RING = B_STAGES * B_BYTES, RAW_RING = A_RING + A_STAGES * A_BYTES;
constexpr int RING_BYTES = RAW_RING + RAW_STAGES * RAW_BYTES;
constexpr int DEQ_GROUPS = 3, DEQ_GROUP_WARPS = 4;
// Warp roles are laid out by scheduler (warp id % 4 selects the SM sub-partition): the two single-thread roles that
// pace the pipeline, TMA (warp 0) and MMA (warp 4), share sub-partition 0 with only one epilogue warp, so the
// instruction-heavy dequantisation warps (sub-partitions 1-3) never compete with them for issue slots.
constexpr int TMA_WARP = 0, MMA_WARP = 4;
constexpr int NUM_WARPS = 20;
constexpr int THREADS = NUM_WARPS * 32;
// epilogue: warps 8 (TMEM lanes 0-31), 1, 2, 3; dequant: the twelve warps >= 5 off sub-partition 0; warps 12, 16 idle
__device__ __forceinline__ bool is_epilogue_warp(int w) { return w == 8 || (w >= 1 && w <= 3); }
__device__ __forceinline__ int dequant_index(int w) {  // 0..11, or -1
    if ((w & 3) == 0 || w < 5) return -1;
    return (w - 5) - ((w - 4) >> 2);  // skip the warps of sub-partition 0 (8, 12, 16)
}
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = RING_BYTES + 1024 + 512;

struct Bars {
    unsigned long long a_full[STAGES], b_full[STAGES], empty[STAGES], raw_full[RAW_STAGES], raw_empty[RAW_STAGES];
    unsigned long long acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    unsigned int abort_flag;
};

struct Params {
    const uint16_t* scales;     // bf16 [weight rows][K / group]
    void* y;                    // [rows][ldy] bf16 or f32
    const uint32_t* m_tiles_dev;  // optional: number of 256-row tiles decided on the device (grouped launches)
    const uint32_t* tile_expert;  // optional: expert of each 256-row tile
    uint32_t* status;
    uint32_t M, N, K, group;    // M: activation/output rows; N: output columns
    uint32_t bn;                // accumulator columns per tile
    uint32_t m_tiles, n_tiles;
    uint32_t expert_rows;       // weight rows per expert in the stacked weight tensor
    uint32_t glu_stride;        // glu: rows between W1[j] and W3[j] of one expert
    uint32_t ldy;               // output row stride in elements
    uint32_t out_f32;           // plain mode only: store f32 instead of bf16
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
// one byte (two nibbles, k even in the low one) -> two bf16 (k, k+1) = bf16((q - 8) * s), natural order
__device__ __forceinline__ uint32_t dequant_byte(uint32_t byte_in_low, uint32_t s2) {
    // 0x1001 spreads the byte so that the low nibble sits at bits 0-3 and the high nibble at bits 16-19
    const uint32_t t = ((byte_in_low * 0x1001u) & 0x000F000Fu) | 0x43004300u;  // (128 + q_k, 128 + q_k+1) exactly
    return bf16x2_mul(bf16x2_sub(t, 0x43084308u), s2);                            // exact q - 8, one rounding of the product
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct TileCoord {
    uint32_t mt, nt, expert;
};

template <bool GLU>
__global__ void __launch_bounds__(THREADS, 1)
int4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    Bars* bars = reinterpret_cast<Bars*>(tiles + RING_BYTES);
    volatile unsigned int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t m_tiles = p.m_tiles_dev ? min(*p.m_tiles_dev, p.m_tiles) : p.m_tiles;
    const uint32_t total_tiles = m_tiles * p.n_tiles, k_blocks = p.K / BK;
    const uint32_t groups = p.K / p.group;
    const uint32_t half_rows = p.bn >> 1;           // weight rows this CTA dequantises per tile
    const uint32_t raw_bytes = half_rows * RAW_KB * (BK / 2);
    const uint32_t raw_blocks = k_blocks / RAW_KB;  // packed-weight loads per tile
    const uint32_t out_cols = GLU ? half_rows : p.bn;  // output columns per tile

    auto coord = [&](uint32_t tile) {
        TileCoord c;
        c.mt = tile % m_tiles;
        c.nt = tile / m_tiles;
        c.expert = p.tile_expert ? p.tile_expert[c.mt] : 0u;
        return c;
    };
    // first weight row (in the stacked tensor) of this CTA's half of a tile
    auto weight_row0 = [&](const TileCoord& c) {
        return GLU ? c.expert * p.expert_rows + rank * p.glu_stride + c.nt * half_rows
                   : c.expert * p.expert_rows + c.nt * p.bn + rank * half_rows;
    };
    // how many of this CTA's weight rows exist (tail tiles in N)
    auto weight_rows_valid = [&](const TileCoord& c) {
        const uint32_t first = GLU ? c.nt * half_rows : c.nt * p.bn + rank * half_rows;
        return first >= p.N ? 0u : min(half_rows, p.N - first);
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->a_full[s]), 1);                    // leader: one expect_tx arrival, bytes from both CTAs
            mbar_init(smem_u32(&bars->b_full[s]), 2 * DEQ_GROUP_WARPS);  // leader: dequant warps of both CTAs
            mbar_init(smem_u32(&bars->empty[s]), 1);                     // one tcgen05.commit per CTA
        }
        for (int s = 0; s < RAW_STAGES; ++s) {
            mbar_init(smem_u32(&bars->raw_full[s]), 1);
            mbar_init(smem_u32(&bars->raw_empty[s]), RAW_KB * DEQ_GROUP_WARPS);  // each stage: the four warps of one group
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars->acc_full[a]), 1);
            mbar_init(smem_u32(&bars->acc_empty[a]), 8);  // leader: 4 epilogue warps of each CTA
        }
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&map_x);
        tma_prefetch_desc(&map_w);
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(smem_u32(&bars->tmem_base), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before any remote arrive, commit or TMA completion can target them
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    const int deq_idx = dequant_index(warp);
    if (warp == TMA_WARP) {
        // ------------------------------------ TMA producer ------------------------------------
        uint32_t a_it = 0, r_it = 0, r_tile = pair, r_blk = 0;
        bool ok = true;
        for (uint32_t tile = pair; tile < total_tiles && ok; tile += pairs) {
            const TileCoord c = coord(tile);
            const int m0 = int(c.mt * 2 * BM + rank * BM);
            for (uint32_t kb = 0; kb < k_blocks && ok; ++kb, ++a_it) {
                while (ok && r_tile < total_tiles && r_it <= a_it / RAW_KB + RAW_AHEAD) {
                    const uint32_t rs = r_it % RAW_STAGES;
                    if (r_it >= RAW_STAGES)
                        ok = mbar_wait(smem_u32(&bars->raw_empty[rs]), ((r_it / RAW_STAGES) - 1) & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    if (lane == 0) {
                        const uint32_t bar = smem_u32(&bars->raw_full[rs]);
                        mbar_arrive_expect_tx(bar, raw_bytes);
                        tma_load_2d(smem_u32(tiles + RAW_RING + rs * RAW_BYTES), &map_w, int(r_blk * RAW_KB * (BK / 2)),
                                    int(weight_row0(coord(r_tile))), bar);
                    }
                    __syncwarp();
                    ++r_it;
                    if (++r_blk == raw_blocks) {
                        r_blk = 0;
                        r_tile += pairs;
                    }
                }
                if (!ok) break;
                const uint32_t as = a_it % A_STAGES;
                if (a_it >= A_STAGES) ok = mbar_wait(smem_u32(&bars->empty[as]), ((a_it / A_STAGES) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (lane == 0) {
                    // both CTAs' activation boxes count on the leader's barrier; the leader posts the expectation
                    const uint32_t leader_bar = mapa(smem_u32(&bars->a_full[as]), 0);
                    if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bars->a_full[as]), 2 * A_BYTES);
                    tma_load_2d_pair(smem_u32(tiles + A_RING + as * A_BYTES), &map_x, int(kb * BK), m0, leader_bar);
                }
                __syncwarp();
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------ MMA issuer (leader CTA only) ------------------------------------
        if (rank == 0) {
            const uint32_t idesc = idesc_bf16_f32(2 * BM, p.bn);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (uint32_t tile = pair; tile < total_tiles && ok; tile += pairs, ++local) {
                const uint32_t acc = local & 1;
                if (local >= 2) ok = mbar_wait(smem_u32(&bars->acc_empty[acc]), ((local >> 1) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * MAX_BN;
                for (uint32_t kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t as = it % A_STAGES, bs = it % B_STAGES;
                    ok = mbar_wait(smem_u32(&bars->a_full[as]), (it / A_STAGES) & 1, abort_flag);
                    ok = ok && mbar_wait(smem_u32(&bars->b_full[bs]), (it / B_STAGES) & 1, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
                    if (lane == 0) {
                        const uint64_t da = smem_desc_sw128(smem_u32(tiles + A_RING + as * A_BYTES));
                        const uint64_t db = smem_desc_sw128(smem_u32(tiles + B_RING + bs * B_BYTES));
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            mma_f16_pair(d_tmem, smem_desc_advance(da, k * UMMA_K * 2), smem_desc_advance(db, k * UMMA_K * 2),
                                         idesc, (kb | uint32_t(k)) != 0);
                        // free the stage in both CTAs
                        const uint32_t em = smem_u32(&bars->empty[as]);
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
        // ------------------------------------ epilogue warps ------------------------------------
        const uint32_t quad = warp & 3;  // TMEM lane quarter this warp may read
        uint32_t local = 0;
        bool ok = true;
        for (uint32_t tile = pair; tile < total_tiles && ok; tile += pairs, ++local) {
            const uint32_t acc = local & 1;
            const TileCoord c = coord(tile);
            ok = mbar_wait(smem_u32(&bars->acc_full[acc]), (local >> 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t row = c.mt * 2 * BM + rank * BM + quad * 32 + lane;
            const uint32_t taddr = tmem_base + ((quad * 32) << 16) + acc * MAX_BN;
            const uint32_t n0 = c.nt * out_cols;
            for (uint32_t cc = 0; cc < out_cols / 32; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + cc * 32, r);
                if constexpr (GLU) {
                    uint32_t ru[32];
                    tmem_ld_32x32(taddr + half_rows + cc * 32, ru);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        // same rounding points as the single-token reference ops: g and u are bf16 values, the
                        // activation is evaluated in f32 as g * (u * (1 / (1 + exp(-g)))) and stored as bf16
                        const float g = bf16_round(__uint_as_float(r[j])), u = bf16_round(__uint_as_float(ru[j]));
                        const float sig = 1.0f / (1.0f + expf(-g));
                        r[j] = __float_as_uint(g * (u * sig));
                    }
                } else {
                    tmem_ld_wait();
                }
                const uint32_t col0 = n0 + cc * 32;
                if (row < p.M && col0 < p.N) {
                    const bool f32_out = !GLU && p.out_f32 != 0;
                    if (f32_out) {
                        float* dst = static_cast<float*>(p.y) + size_t(row) * p.ldy + col0;
                        if (col0 + 32 <= p.N && (p.ldy & 3u) == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4*>(dst)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < p.N) dst[j] = __uint_as_float(r[j]);
                        }
                    } else {
                        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.y) + size_t(row) * p.ldy + col0;
                        if (col0 + 32 <= p.N && (p.ldy & 7u) == 0) {
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
                                if (col0 + j < p.N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&bars->acc_empty[acc]), 0));
        }
    } else if (deq_idx >= 0) {
        // ------------------------------------ dequant warps ------------------------------------
        const uint32_t dgroup = uint32_t(deq_idx) / DEQ_GROUP_WARPS;  // takes the stages with stage % DEQ_GROUPS == dgroup
        const uint32_t r = (uint32_t(deq_idx) % DEQ_GROUP_WARPS) * 32 + lane;  // weight row of this thread
        const uint32_t gdiv = p.group / BK;            // stages per scale group
        uint32_t it_base = 0, raw_base = 0;
        bool ok = true;
        for (uint32_t tile = pair; tile < total_tiles && ok; tile += pairs, raw_base += raw_blocks, it_base += k_blocks) {
            const TileCoord c = coord(tile);
            const bool row_valid = r < weight_rows_valid(c);
            const uint16_t* srow = p.scales + size_t(row_valid ? weight_row0(c) + r : 0) * groups;
            // Each stage needs one group scale per row. The loads run four of this warp's stages ahead (a queue of
            // four registers): one stage ahead is not enough, an L2 hit costs more than a stage takes.
            // this group's stages of the tile: global stage numbers congruent to dgroup modulo DEQ_GROUPS
            const uint32_t kb_first = (dgroup + DEQ_GROUPS - it_base % DEQ_GROUPS) % DEQ_GROUPS;
            const uint32_t n_own = kb_first < k_blocks ? (k_blocks - kb_first + DEQ_GROUPS - 1) / DEQ_GROUPS : 0u;
            uint32_t q[4];
#pragma unroll
            for (uint32_t d = 0; d < 4; ++d)
                q[d] = (row_valid && d < n_own) ? uint32_t(srow[(kb_first + DEQ_GROUPS * d) / gdiv]) : 0u;
            for (uint32_t j0 = 0; j0 < n_own && ok; j0 += 4) {
#pragma unroll
              for (uint32_t u = 0; u < 4; ++u) {
                const uint32_t j = j0 + u;
                if (j >= n_own || !ok) break;
                const uint32_t kb = DEQ_GROUPS * j + kb_first, it = it_base + kb;
                const uint32_t r_it = raw_base + kb / RAW_KB, rs = r_it % RAW_STAGES, bs = it % B_STAGES;
                const uint32_t sv = q[u];
                const uint32_t s2 = sv | (sv << 16);  // this stage's group scale in both bf16 halves
                if (row_valid && j + 4 < n_own) q[u] = uint32_t(srow[(kb + 4 * DEQ_GROUPS) / gdiv]);
                ok = mbar_wait(smem_u32(&bars->raw_full[rs]), (r_it / RAW_STAGES) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                // the packed slot holds 128-byte rows (4 k-blocks) with the 128-byte swizzle: 16-byte chunk c of row r
                // sits at chunk c ^ (r & 7), which also keeps a quarter warp's reads in distinct bank groups
                const uint8_t* raw_row = tiles + RAW_RING + rs * RAW_BYTES + r * 128;
                const uint32_t c0 = (kb % RAW_KB) * 2;
                uint4 w0 = make_uint4(0, 0, 0, 0), w1 = w0;
                if (r < half_rows) {
                    w0 = *reinterpret_cast<const uint4*>(raw_row + ((c0 ^ (r & 7u)) << 4));
                    w1 = *reinterpret_cast<const uint4*>(raw_row + (((c0 + 1) ^ (r & 7u)) << 4));
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->raw_empty[rs]));  // the packed bytes now live in registers
                const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                uint4 o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t w = words[j];
                    o[j].x = dequant_byte(w & 0xFFu, s2);
                    o[j].y = dequant_byte(__byte_perm(w, 0, 0x4441), s2);
                    o[j].z = dequant_byte(__byte_perm(w, 0, 0x4442), s2);
                    o[j].w = dequant_byte(w >> 24, s2);
                }
                // the dequantised slot must have been consumed by the MMAs of its previous use
                if (it >= B_STAGES) ok = mbar_wait(smem_u32(&bars->empty[bs]), ((it / B_STAGES) - 1) & 1, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (r < half_rows) {
                    uint8_t* brow = tiles + B_RING + bs * B_BYTES + r * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) *reinterpret_cast<uint4*>(brow + ((uint32_t(j) ^ (r & 7u)) << 4)) = o[j];
                }
                fence_proxy_async();  // generic-proxy stores -> visible to the tensor core's operand reads
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&bars->b_full[bs]), 0));
              }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer may still be reading this CTA's shared memory / TMEM through the pair MMA until here
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
    if (threadIdx.x == 0 && bars->abort_flag != 0 && p.status) atomicOr(p.status, 16u);
}

}  // namespace

bool int4_gemm_pair_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    // 64-k stages must not straddle a scale group; packed weights are fetched 256 k at a time; one CTA pair per
    // 256 activation rows only pays above 128 rows
    return m > 128 && n >= 1 && k >= 256 && k % 256 == 0 && group >= 64 && group % 64 == 0 && k % group == 0;
}

namespace {

// accumulator columns per tile
uint32_t choose_bn(uint32_t n, bool glu) {
    // 256 accumulator columns amortise the activation operand best (measured: 224-wide tiles are slower even when
    // they save a tail wave); narrower tiles only when the problem itself is narrow
    const uint32_t cols = glu ? 2 * n : n;
    const uint32_t step = glu ? 64 : 32;
    uint32_t bn = ((cols + step - 1) / step) * step;
    if (bn < 128) bn = 128;
    if (bn > 256) bn = 256;
    return bn;
}

}  // namespace

cudaError_t launch_int4_gemm_pair(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                  uint32_t n, uint32_t k, uint32_t group, uint32_t out_f32, uint32_t glu, uint32_t experts,
                                  const uint32_t* tile_expert, const uint32_t* m_tiles_dev, uint32_t ldy, int sm_count,
                                  cudaStream_t stream, uint32_t* status) {
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load() & bit)) {
        e = cudaFuncSetAttribute(int4_gemm_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(int4_gemm_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit);
    }
    if (experts == 0) experts = 1;
    const uint32_t pairs_avail = uint32_t(sm_count) / 2;
    if (pairs_avail == 0) return cudaErrorInvalidConfiguration;
    Params p{};
    p.m_tiles = (m + 2 * BM - 1) / (2 * BM);
    p.bn = choose_bn(n, glu != 0);
    // Few tiles (a decode-sized batch, or one expert's rows on an expert-parallel rank): with 256-wide tiles a handful of
    // tiles beyond one wave of CTA pairs costs a whole second wave (5 row tiles x 16 column tiles = 80 tiles on 74 pairs
    // is two waves). 128-wide tiles halve that granularity; they amortise the activation operand less well, which only
    // matters once there are many waves.
    if (!glu && p.bn == 256 && uint64_t(p.m_tiles) * ((n + 255) / 256) < 4ull * pairs_avail) p.bn = 128;
    const uint32_t cols = glu ? p.bn / 2 : p.bn;
    p.n_tiles = (n + cols - 1) / cols;
    p.scales = static_cast<const uint16_t*>(scale_bf16);
    p.y = y;
    p.m_tiles_dev = m_tiles_dev;
    p.tile_expert = tile_expert;
    p.status = status;
    p.M = m;
    p.N = n;
    p.K = k;
    p.group = group;
    p.expert_rows = glu ? 2 * n : n;
    p.glu_stride = n;
    p.ldy = ldy;
    p.out_f32 = out_f32;
    const uint64_t weight_rows = uint64_t(experts) * p.expert_rows;
    CUtensorMap mx, mw;
    if (!encode_tensor_map_2d(&mx, x_bf16, m, k, 2, BM, BK, true) ||
        !encode_tensor_map_2d(&mw, w_packed, weight_rows, k / 2, 1, p.bn / 2, RAW_KB * (BK / 2), true))
        return cudaErrorInvalidValue;
    const uint32_t tiles = p.m_tiles * p.n_tiles;
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
    if (glu)
        e = cudaLaunchKernelEx(&cfg, int4_gemm_pair_kernel<true>, mx, mw, p);
    else
        e = cudaLaunchKernelEx(&cfg, int4_gemm_pair_kernel<false>, mx, mw, p);
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace vybk

