// Decode GEMV / skinny GEMM for group-quantized int4 weights (batch <= 8 per pass), sm_100a.
//
//   y[m, n] = cast( sum_k x[m, k] * (q[n, k] - 8) * s[n, k / 128] )      f32 accumulate
//
// The op is HBM-bound: 0.5 byte of weight per MAC and nothing is reused, so the design goal is to keep
// ~35 KB of loads in flight per SM and to spend as few issue slots per weight as possible.
//
//  * One persistent CTA per SM owns a contiguous row range of W (balanced to within one row).
//  * A producer warp streams the range in 16-row x 4096-k stages with 1-D bulk TMA copies
//    (cp.async.bulk, one 2 KB copy per row, one 64 B copy per row of scales) into a 4-stage shared-memory
//    ring guarded by full/empty mbarriers: 4 x 35 KB in flight per SM, DRAM sees purely sequential streams.
//    Row pitch in shared memory is 2048+64 B so that the 128-bit fragment loads below are bank-conflict free.
//  * 16 consumer warps each own a fixed 256-k slice of the stage. The activation fragments for that slice
//    live in registers for the whole kernel (32 regs), so shared memory is read exactly once per weight byte.
//  * Dequantisation is two instructions per two weights: (w >> 4i) & 0x000F000F | 0x43004300 is the bf16 pair
//    (128+q_lo, 128+q_hi), a packed bf16 subtract of 136 makes it (q_lo-8, q_hi-8) exactly, and the pair is
//    fed straight into mma.sync.m16n8k16 (A = 16 weight rows, B = 8 batch columns, f32 accumulate). k is
//    permuted identically on the A and B side, which a contraction allows. The group scale multiplies the
//    f32 group result, so products are exact and only f32 accumulation rounds.
//  * Each warp leaves a 16x8 partial per tile in a shared slot; the last warp to arrive reduces the 16
//    partials in fixed order (deterministic) and stores the outputs.
//
// Every mbarrier wait is bounded; when a wait runs out the kernel raises a status word and drains instead of
// spinning forever or trapping.
//
// Replaces the generated scalar kernel of vyre-libs/src/nn/linear/inner/linear_4bit.rs:399-775 (one warp per
// output, 4-byte loads, scalar f32 FMA) for the row-major layout of
// vyre-primitives/src/math/quantized/programs.rs:186-300.
#include <cuda_bf16.h>

#include <atomic>

#include "kernels.h"

namespace vybk {
namespace {

constexpr int TILE_ROWS = 16;
constexpr int KBLOCK = 4096;
constexpr int CONSUMER_WARPS = 16;
constexpr int WARP_K = KBLOCK / CONSUMER_WARPS;  // 256 = two 128-k groups
constexpr int STAGES = 4;
constexpr int ROW_BYTES = KBLOCK / 2;
constexpr int ROW_PITCH = ROW_BYTES + 64;
constexpr int SCALE_ROW_BYTES = (KBLOCK / 128) * 2;
constexpr int SCALE_PITCH = 80;
constexpr int STAGE_W_BYTES = TILE_ROWS * ROW_PITCH;
constexpr int STAGE_S_BYTES = TILE_ROWS * SCALE_PITCH;
constexpr int STAGE_BYTES = STAGE_W_BYTES + STAGE_S_BYTES;
constexpr int RED_SLOTS = 2 * STAGES;
constexpr int RED_SLOT_FLOATS = CONSUMER_WARPS * 128;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int SMEM_RING = STAGES * STAGE_BYTES;
constexpr int SMEM_RED = RED_SLOTS * RED_SLOT_FLOATS * 4;
constexpr int SMEM_CTRL = 256;
constexpr int SMEM_TOTAL = SMEM_RING + SMEM_RED + SMEM_CTRL;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr long long WAIT_CLOCKS = 2000000000ll;  // about a second at boost clocks

static_assert(STAGE_BYTES % 128 == 0, "stage must stay 128-byte aligned");
static_assert(SMEM_TOTAL <= 232448, "shared memory budget");

struct Ctrl {
    unsigned long long full[STAGES];
    unsigned long long empty[STAGES];
    unsigned int count[RED_SLOTS];
    unsigned int abort_flag;
};
static_assert(sizeof(Ctrl) <= SMEM_CTRL, "control block");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another warp already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile unsigned int* abort_flag) {
    const long long t0 = clock64();
    for (uint32_t it = 0; it < WAIT_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u && (*abort_flag != 0 || clock64() - t0 > WAIT_CLOCKS)) break;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// bf16 pair (nibble i - 8, nibble i+4 - 8) of a packed word: the LOP3 builds (128+q) in both halves, the packed
// subtract of 136 (0x4308) is exact
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, int i) {
    const uint32_t v = ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
    uint32_t r;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(0x43084308u));
    return r;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

struct Params {
    const uint16_t* x;
    const uint8_t* w;
    const uint16_t* scales;
    void* y;
    uint32_t m, n, k, groups;  // groups = k / 128
    uint32_t out_f32;
    uint32_t* status;
    unsigned long long* trace;  // optional: per-CTA timeline (64 slots each), for tuning only
};

__global__ void __launch_bounds__(THREADS, 1) int4_gemv_kernel(const Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    float* red = reinterpret_cast<float*>(smem + SMEM_RING);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + SMEM_RING + SMEM_RED);
    volatile unsigned int* abort_flag = &ctrl->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    auto stamp = [&](int slot) {
        if (p.trace && lane == 0 && (warp == 0 || warp == CONSUMER_WARPS)) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            p.trace[size_t(blockIdx.x) * 64 + (warp == 0 ? 0 : 32) + slot] = t;
        }
    };
    stamp(0);
    const uint32_t r0 = uint32_t((uint64_t(blockIdx.x) * p.n) / gridDim.x);
    const uint32_t r1 = uint32_t((uint64_t(blockIdx.x + 1) * p.n) / gridDim.x);
    const uint32_t ntiles = (r1 - r0 + TILE_ROWS - 1) / TILE_ROWS;
    const uint32_t nkb = (p.k + KBLOCK - 1) / KBLOCK;
    const uint32_t units = ntiles * nkb;
    const uint32_t row_bytes = p.k / 2;
    // When one k-block covers the whole row (k <= 4096) the rows of a tile are contiguous in global memory:
    // the whole tile is ONE bulk copy (and its scales one more), laid out in shared memory with the global
    // pitch. Otherwise each row needs its own copy and gets a padded, bank-conflict-free pitch.
    const bool contiguous = nkb == 1;
    const uint32_t row_pitch = contiguous ? row_bytes : uint32_t(ROW_PITCH);
    const uint32_t scale_pitch = contiguous ? p.groups * 2 : uint32_t(SCALE_PITCH);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);
            mbar_init(smem_u32(&ctrl->empty[s]), CONSUMER_WARPS);
        }
        for (int s = 0; s < RED_SLOTS; ++s) ctrl->count[s] = 0;
        ctrl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    stamp(1);

    if (warp == CONSUMER_WARPS) {
        // ------------------------------ producer warp ------------------------------
        bool alive = true;
        for (uint32_t u = 0; u < units && alive; ++u) {
            const uint32_t s = u % STAGES;
            if (u >= STAGES) alive = mbar_wait(smem_u32(&ctrl->empty[s]), ((u / STAGES) - 1) & 1, abort_flag);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            const uint32_t tile = u / nkb, kb = u % nkb;
            const uint32_t row_base = r0 + tile * TILE_ROWS;
            const uint32_t rows_valid = min(uint32_t(TILE_ROWS), r1 - row_base);
            const uint32_t kbytes = min(uint32_t(KBLOCK), p.k - kb * KBLOCK) / 2;
            const uint32_t sbytes = min(uint32_t(KBLOCK / 128), p.groups - kb * (KBLOCK / 128)) * 2;
            const uint32_t bar = smem_u32(&ctrl->full[s]);
            if (u < 12) stamp(2 + u);
            uint8_t* stage = ring + size_t(s) * STAGE_BYTES;
            if (contiguous) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(bar, rows_valid * (kbytes + sbytes));
                    bulk_g2s(smem_u32(stage), p.w + size_t(row_base) * row_bytes, rows_valid * kbytes, bar);
                    bulk_g2s(smem_u32(stage + STAGE_W_BYTES), p.scales + size_t(row_base) * p.groups,
                             rows_valid * sbytes, bar);
                }
            } else {
                if (lane == 0) mbar_arrive_expect_tx(bar, rows_valid * (kbytes + sbytes));
                __syncwarp();
                if (lane < TILE_ROWS) {
                    if (uint32_t(lane) < rows_valid)
                        bulk_g2s(smem_u32(stage + lane * ROW_PITCH),
                                 p.w + size_t(row_base + lane) * row_bytes + size_t(kb) * ROW_BYTES, kbytes, bar);
                } else {
                    const uint32_t r = lane - TILE_ROWS;
                    if (r < rows_valid)
                        bulk_g2s(smem_u32(stage + STAGE_W_BYTES + r * SCALE_PITCH),
                                 p.scales + size_t(row_base + r) * p.groups + size_t(kb) * (KBLOCK / 128), sbytes,
                                 bar);
                }
            }
            __syncwarp();
        }
        if (!alive && lane == 0 && p.status) atomicOr(p.status, 1u);
        return;
    }

    // -------------------------------- consumer warps --------------------------------
    const int g = lane >> 2;  // mma row group / batch column of the B fragment
    const int t = lane & 3;
    uint32_t xb[2][4][4];

    auto load_x = [&](uint32_t kb) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const uint32_t k0 = kb * KBLOCK + warp * WARP_K + c * 128 + t * 32 + wi * 8;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (uint32_t(g) < p.m && k0 < p.k) v = *reinterpret_cast<const uint4*>(p.x + size_t(g) * p.k + k0);
                xb[c][wi][0] = __byte_perm(v.x, v.z, 0x5410);  // (x0, x4)
                xb[c][wi][1] = __byte_perm(v.x, v.z, 0x7632);  // (x1, x5)
                xb[c][wi][2] = __byte_perm(v.y, v.w, 0x5410);  // (x2, x6)
                xb[c][wi][3] = __byte_perm(v.y, v.w, 0x7632);  // (x3, x7)
            }
        }
    };
    if (nkb == 1) load_x(0);
    stamp(2);

    // per-unit register image of this warp's slice of the stage: 2 x 16 B of each of the two fragment rows
    // plus the two group scales of each row
    struct Frag {
        uint4 wl[2], wh[2];
        uint32_t sc_lo, sc_hi;
    };
    auto fetch = [&](uint32_t u, Frag& f) -> bool {
        const uint32_t s = u % STAGES;
        bool ok = mbar_wait(smem_u32(&ctrl->full[s]), (u / STAGES) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return false;
        const uint8_t* stage = ring + size_t(s) * STAGE_BYTES;
        const uint8_t* wrow_lo = stage + g * row_pitch + warp * (WARP_K / 2) + t * 16;
        const uint8_t* wrow_hi = wrow_lo + 8 * row_pitch;
        f.wl[0] = *reinterpret_cast<const uint4*>(wrow_lo);
        f.wh[0] = *reinterpret_cast<const uint4*>(wrow_hi);
        f.wl[1] = *reinterpret_cast<const uint4*>(wrow_lo + 64);
        f.wh[1] = *reinterpret_cast<const uint4*>(wrow_hi + 64);
        f.sc_lo = *reinterpret_cast<const uint32_t*>(stage + STAGE_W_BYTES + g * scale_pitch + warp * 4);
        f.sc_hi = *reinterpret_cast<const uint32_t*>(stage + STAGE_W_BYTES + (g + 8) * scale_pitch + warp * 4);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->empty[s]));
        return true;
    };

    Frag cur, nxt;
    bool alive = units > 0 ? fetch(0, cur) : true;
    for (uint32_t tile = 0; tile < ntiles && alive; ++tile) {
        float out[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t kb = 0; kb < nkb; ++kb) {
            const uint32_t u = tile * nkb + kb;
            if (nkb != 1) load_x(kb);
            if (u < 12) stamp(3 + 2 * u);
            // software pipeline: pull the next unit's fragments into registers before the math of this one
            const bool have_next = u + 1 < units;
            if (have_next && nkb == 1) {
                alive = fetch(u + 1, nxt);
                if (!alive) break;
            }
            if (kb * KBLOCK + warp * WARP_K < p.k) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    // two independent accumulator chains per group keep the tensor pipe from waiting on itself
                    float acc0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    float acc1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    const uint32_t lo[4] = {cur.wl[c].x, cur.wl[c].y, cur.wl[c].z, cur.wl[c].w};
                    const uint32_t hi[4] = {cur.wh[c].x, cur.wh[c].y, cur.wh[c].z, cur.wh[c].w};
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi) {
                        mma_bf16(acc0, nib_pair(lo[wi], 0), nib_pair(hi[wi], 0), nib_pair(lo[wi], 1), nib_pair(hi[wi], 1),
                                 xb[c][wi][0], xb[c][wi][1]);
                        mma_bf16(acc1, nib_pair(lo[wi], 2), nib_pair(hi[wi], 2), nib_pair(lo[wi], 3), nib_pair(hi[wi], 3),
                                 xb[c][wi][2], xb[c][wi][3]);
                    }
                    const float s_lo = c == 0 ? bf16_lo(cur.sc_lo) : bf16_hi(cur.sc_lo);
                    const float s_hi = c == 0 ? bf16_lo(cur.sc_hi) : bf16_hi(cur.sc_hi);
                    out[0] = fmaf(s_lo, acc0[0] + acc1[0], out[0]);
                    out[1] = fmaf(s_lo, acc0[1] + acc1[1], out[1]);
                    out[2] = fmaf(s_hi, acc0[2] + acc1[2], out[2]);
                    out[3] = fmaf(s_hi, acc0[3] + acc1[3], out[3]);
                }
            }
            if (have_next) {
                if (nkb == 1) {
                    cur = nxt;
                } else {
                    alive = fetch(u + 1, cur);
                    if (!alive) break;
                }
            }
        }
        if (!alive) break;
        if (tile < 12) stamp(4 + 2 * tile);

        // cross-warp reduction of the tile: last arriving warp sums the 16 partials in warp order
        const uint32_t slot = tile % RED_SLOTS;
        float* slot_base = red + size_t(slot) * RED_SLOT_FLOATS;
        *reinterpret_cast<float4*>(slot_base + warp * 128 + lane * 4) = make_float4(out[0], out[1], out[2], out[3]);
        __threadfence_block();
        __syncwarp();
        unsigned int old = 0;
        if (lane == 0) old = atomicAdd(&ctrl->count[slot], 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == CONSUMER_WARPS - 1) {
            __threadfence_block();
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < CONSUMER_WARPS; ++w) {
                const float4 v = *reinterpret_cast<const float4*>(slot_base + w * 128 + lane * 4);
                sum.x += v.x;
                sum.y += v.y;
                sum.z += v.z;
                sum.w += v.w;
            }
            __syncwarp();
            if (lane == 0) ctrl->count[slot] = 0;
            const uint32_t row_lo = r0 + tile * TILE_ROWS + g;
            const uint32_t row_hi = row_lo + 8;
            const uint32_t n0 = 2 * t, n1 = 2 * t + 1;
            if (p.out_f32) {
                float* y = static_cast<float*>(p.y);
                if (row_lo < r1) {
                    if (n0 < p.m) y[size_t(n0) * p.n + row_lo] = sum.x;
                    if (n1 < p.m) y[size_t(n1) * p.n + row_lo] = sum.y;
                }
                if (row_hi < r1) {
                    if (n0 < p.m) y[size_t(n0) * p.n + row_hi] = sum.z;
                    if (n1 < p.m) y[size_t(n1) * p.n + row_hi] = sum.w;
                }
            } else {
                __nv_bfloat16* y = static_cast<__nv_bfloat16*>(p.y);
                if (row_lo < r1) {
                    if (n0 < p.m) y[size_t(n0) * p.n + row_lo] = __float2bfloat16_rn(sum.x);
                    if (n1 < p.m) y[size_t(n1) * p.n + row_lo] = __float2bfloat16_rn(sum.y);
                }
                if (row_hi < r1) {
                    if (n0 < p.m) y[size_t(n0) * p.n + row_hi] = __float2bfloat16_rn(sum.z);
                    if (n1 < p.m) y[size_t(n1) * p.n + row_hi] = __float2bfloat16_rn(sum.w);
                }
            }
        }
    }
    stamp(31);
    if (!alive && lane == 0 && p.status) atomicOr(p.status, 2u);
}

// ---- fallback: any group size dividing k, any batch; warp per output row, plain 32-bit loads -------------------
__global__ void __launch_bounds__(256) int4_linear_generic_kernel(const uint16_t* __restrict__ x,
                                                                 const uint32_t* __restrict__ w,
                                                                 const uint16_t* __restrict__ scales, void* y,
                                                                 uint32_t m, uint32_t n, uint32_t k, uint32_t group,
                                                                 uint32_t out_f32) {
    const uint32_t row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (row >= n) return;
    const uint32_t words = k / 8, groups = k / group;
    for (uint32_t b0 = 0; b0 < m; b0 += 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (uint32_t wi = lane; wi < words; wi += 32) {
            const uint32_t word = w[size_t(row) * words + wi];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t kk = wi * 8 + i;
                const float s = __uint_as_float(uint32_t(scales[size_t(row) * groups + kk / group]) << 16);
                const float wv = float(int((word >> (4 * i)) & 0xF) - 8) * s;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (b0 + j < m) acc[j] = fmaf(__uint_as_float(uint32_t(x[size_t(b0 + j) * k + kk]) << 16), wv, acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v = acc[j];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && b0 + j < m) {
                if (out_f32)
                    static_cast<float*>(y)[size_t(b0 + j) * n + row] = v;
                else
                    static_cast<__nv_bfloat16*>(y)[size_t(b0 + j) * n + row] = __float2bfloat16_rn(v);
            }
        }
    }
}

}  // namespace

unsigned long long* g_gemv_trace = nullptr;
void set_int4_gemv_trace(unsigned long long* t) { g_gemv_trace = t; }

bool int4_gemv_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    return m >= 1 && m <= 8 && n >= 1 && group == 128 && k >= 1024 && k % 1024 == 0;
}

cudaError_t launch_int4_gemv(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                             uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                             uint32_t* status) {
    // opt in to the large dynamic shared-memory carve-out once per device
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t de = cudaGetDevice(&dev);
    if (de != cudaSuccess) return de;
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(int4_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit, std::memory_order_release);
    }
    Params p;
    p.x = static_cast<const uint16_t*>(x_bf16);
    p.w = static_cast<const uint8_t*>(w_packed);
    p.scales = static_cast<const uint16_t*>(scale_bf16);
    p.y = y;
    p.m = m;
    p.n = n;
    p.k = k;
    p.groups = k / 128;
    p.out_f32 = out_f32;
    p.status = status;
    p.trace = g_gemv_trace;
    const uint32_t tiles = (n + TILE_ROWS - 1) / TILE_ROWS;
    const uint32_t grid = tiles < uint32_t(sm_count) ? tiles : uint32_t(sm_count);
    int4_gemv_kernel<<<grid, THREADS, SMEM_TOTAL, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_int4_linear_generic(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y,
                                       uint32_t m, uint32_t n, uint32_t k, uint32_t group, uint32_t out_f32,
                                       cudaStream_t stream) {
    int4_linear_generic_kernel<<<(n + 7) / 8, 256, 0, stream>>>(
        static_cast<const uint16_t*>(x_bf16), static_cast<const uint32_t*>(w_packed),
        static_cast<const uint16_t*>(scale_bf16), y, m, n, k, group, out_f32);
    return cudaGetLastError();
}

}  // namespace vybk
