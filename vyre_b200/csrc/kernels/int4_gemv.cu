// Decode GEMV / skinny GEMM for group-quantized int4 weights (batch <= 8 per pass), sm_100a.
//
//   y[m, n] = cast( sum_k x[m, k] * (q[n, k] - 8) * s[n, k / 128] )
//
// The op is HBM-bound (0.5 byte of weight per MAC, nothing reused), so the kernel is built around two
// budgets: keep tens of KB of loads in flight per SM, and spend as few issue slots per weight as possible.
// Integer/logic instructions run at half rate, and a bf16 dequantisation (shift, mask, or-magic, subtract
// per nibble pair) costs more issue time per byte than HBM needs to deliver it, so the weights never become
// floating point here.
//
//  * One persistent CTA per SM owns a contiguous row range of W (balanced to within one row) and streams it
//    in 16-row x 4096-k stages through a 4-stage shared-memory ring guarded by full/empty mbarriers. When a
//    k-block covers the whole row (k <= 4096) the 16 rows of a stage are contiguous in global memory and the
//    stage is ONE 32 KB bulk TMA copy plus one for its scales (cp.async.bulk); per-copy issue cost is what
//    limits a TMA producer, so few large copies matter. Longer rows fall back to one copy per row.
//  * 16 warps each own a fixed 256-k slice of the stage. The activation fragments of that slice live in
//    registers for the whole kernel, so shared memory is read exactly once per weight byte.
//  * A packed word holds 8 nibbles. `(w & 0xF0F0F0F0) ^ 0x80808080` turns the four odd nibbles into the signed
//    bytes 16*(q-8) (a nibble in the high half of a byte with its top bit flipped IS the two's-complement
//    value scaled by 16); `((w << 4) & 0xF0F0F0F0) ^ 0x80808080` does the same for the even ones: 3 logic
//    instructions per 8 weights, zero point included. Those bytes are the A operand of
//    mma.sync.m16n8k32 (s8 x u8/s8, s32 accumulate). k is permuted identically on both operands.
//  * The bf16 activations are converted once per kernel to block-floating integers: per (batch row, 128-k
//    group) a power-of-two step delta = 2^(e_max - 8*LIMBS + 2) and X = rint(x / delta), split into LIMBS
//    byte limbs (low limbs unsigned, top limb signed), each limb its own B operand. bf16 carries 8
//    significant bits, so with LIMBS = 3 every element within 2^-16 of its group's maximum is represented
//    exactly (f32 outputs); LIMBS = 2 keeps 16 bits per group (error <= 2^-16 of the group maximum per
//    element, far inside the 1e-2 window of bf16 outputs). Integer accumulation is exact; per group the limb
//    sums are recombined in f32 and scaled by s * delta / 16, the only place rounding happens.
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
constexpr int WARPS = 16;
constexpr int WARP_K = KBLOCK / WARPS;  // 256 = two 128-k groups
constexpr int STAGES = 4;
constexpr int ROW_BYTES = KBLOCK / 2;
constexpr int ROW_PITCH = ROW_BYTES + 64;  // padded pitch of the per-row copy path (conflict-free fragment loads)
constexpr int SCALE_PITCH = 80;
constexpr int STAGE_W_BYTES = TILE_ROWS * ROW_PITCH;
constexpr int STAGE_S_BYTES = TILE_ROWS * SCALE_PITCH;
constexpr int STAGE_BYTES = STAGE_W_BYTES + STAGE_S_BYTES;
constexpr int RED_SLOTS = 2 * STAGES;
constexpr int RED_SLOT_FLOATS = WARPS * 128;
constexpr int THREADS = (WARPS + 1) * 32;  // 16 consumer warps + 1 producer warp
constexpr int SMEM_RING = STAGES * STAGE_BYTES;
constexpr int X_PITCH = KBLOCK + 16;  // byte pitch of one staged activation row (keeps fragment reads conflict-free)
constexpr int SMEM_RED = RED_SLOTS * RED_SLOT_FLOATS * 4 + 2048;  // reduction slots; doubles as X staging in the prologue
constexpr int SMEM_CTRL = 256;
constexpr int SMEM_TOTAL = SMEM_RING + SMEM_RED + SMEM_CTRL;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr long long WAIT_CLOCKS = 2000000000ll;  // about a second at boost clocks

static_assert(STAGE_BYTES % 128 == 0, "stage must stay 128-byte aligned");
static_assert(SMEM_TOTAL <= 232448, "shared memory budget");

struct Ctrl {
    unsigned long long full[STAGES];
    unsigned long long empty[STAGES];
    unsigned long long red_full[RED_SLOTS];  // 16 arrivals: every warp left its partial of the tile in the slot
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
    if (mbar_try_wait(bar, parity)) return true;
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
// D(16x8, s32) += A(16x32, s8, row) * B(32x8, u8 or s8, col)
template <bool B_SIGNED>
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    if constexpr (B_SIGNED) {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}
// signed bytes 16*(q-8) of the four even / odd nibbles of a packed word
__device__ __forceinline__ uint32_t even_nibbles(uint32_t w) { return ((w << 4) & 0xF0F0F0F0u) ^ 0x80808080u; }
__device__ __forceinline__ uint32_t odd_nibbles(uint32_t w) { return (w & 0xF0F0F0F0u) ^ 0x80808080u; }
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

struct Params {
    const uint16_t* x;
    const uint8_t* w;
    const uint16_t* scales;
    void* y;
    uint32_t m, n, k, groups;  // groups = k / 128
    uint32_t* status;
};

template <int LIMBS, bool OUT_F32>
__global__ void __launch_bounds__(THREADS, 1) int4_gemv_kernel(const Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    float* red = reinterpret_cast<float*>(smem + SMEM_RING);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + SMEM_RING + SMEM_RED);
    volatile unsigned int* abort_flag = &ctrl->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Programmatic dependent launch: let the next kernel in the stream begin its own launch and weight prefetch
    // now; it still waits (griddepcontrol.wait) before touching activations or outputs. No-ops for plain launches.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t rows_base = p.n / gridDim.x, rows_rem = p.n % gridDim.x;
    const uint32_t r0 = blockIdx.x * rows_base + min(blockIdx.x, rows_rem);
    const uint32_t r1 = r0 + rows_base + (blockIdx.x < rows_rem ? 1u : 0u);
    const uint32_t ntiles = (r1 - r0 + TILE_ROWS - 1) / TILE_ROWS;
    const uint32_t nkb = (p.k + KBLOCK - 1) / KBLOCK;
    const uint32_t units = ntiles * nkb;
    const uint32_t row_bytes = p.k / 2;
    // One k-block per row (k <= 4096): the rows of a tile are contiguous in global memory, the whole tile is
    // one bulk copy laid out with the global pitch. Otherwise one copy per row into a padded pitch.
    const bool contiguous = nkb == 1;
    const uint32_t row_pitch = contiguous ? row_bytes : uint32_t(ROW_PITCH);
    const uint32_t scale_pitch = contiguous ? p.groups * 2 : uint32_t(SCALE_PITCH);

    // Producer warp: fill the stage of unit u. Contiguous mode needs lane 0 only.
    auto produce = [&](uint32_t u) {
        const uint32_t s = u % STAGES;
        const uint32_t tile = u / nkb, kb = u % nkb;
        const uint32_t row_base = r0 + tile * TILE_ROWS;
        const uint32_t rows_valid = min(uint32_t(TILE_ROWS), r1 - row_base);
        const uint32_t kbytes = min(uint32_t(KBLOCK), p.k - kb * KBLOCK) / 2;
        const uint32_t sbytes = min(uint32_t(KBLOCK / 128), p.groups - kb * (KBLOCK / 128)) * 2;
        const uint32_t bar = smem_u32(&ctrl->full[s]);
        uint8_t* stage = ring + size_t(s) * STAGE_BYTES;
        if (contiguous) {
            if (lane == 0) {
                mbar_arrive_expect_tx(bar, rows_valid * (kbytes + sbytes));
                bulk_g2s(smem_u32(stage), p.w + size_t(row_base) * row_bytes, rows_valid * kbytes, bar);
                bulk_g2s(smem_u32(stage + STAGE_W_BYTES), p.scales + size_t(row_base) * p.groups, rows_valid * sbytes,
                         bar);
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
                             p.scales + size_t(row_base + r) * p.groups + size_t(kb) * (KBLOCK / 128), sbytes, bar);
            }
            __syncwarp();
        }
    };

    // Whole-row case: the activations are quantised ONCE per CTA, spread over all 512 threads (8 elements per
    // thread per batch row), through a staging area that later becomes the reduction slots. Their loads are
    // issued first of all: behind 140 KB of bulk weight traffic per SM they would wait microseconds.
    const uint32_t stage_bytes_x = uint32_t(LIMBS) * p.m * X_PITCH;
    const bool coop = nkb == 1 && stage_bytes_x + p.m * 32 * 4 <= uint32_t(SMEM_RED);
    uint4 xv[8];
    // activations may come from the preceding kernel: everything that reads x or writes y runs after this point,
    // only the (constant) weight stream of the producer warp starts before it
    if (warp != WARPS) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (coop) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            xv[j] = make_uint4(0, 0, 0, 0);
            if (uint32_t(j) < p.m && threadIdx.x * 8 < p.k)
                xv[j] = *reinterpret_cast<const uint4*>(p.x + size_t(j) * p.k + threadIdx.x * 8);
        }
    }

    if (warp == WARPS) {
        // ------------------------------ producer warp ------------------------------
        if (lane == 0) {
            for (int s = 0; s < STAGES; ++s) {
                mbar_init(smem_u32(&ctrl->full[s]), 1);
                mbar_init(smem_u32(&ctrl->empty[s]), WARPS);
            }
            for (int s = 0; s < RED_SLOTS; ++s) mbar_init(smem_u32(&ctrl->red_full[s]), WARPS);
            ctrl->abort_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        __syncwarp();
        // tell the consumers the barriers exist (they wait on named barrier 2) and start streaming at once
        asm volatile("bar.arrive 2, %0;" ::"n"(THREADS) : "memory");
        bool ok = true;
        for (uint32_t u = 0; u < units; ++u) {
            if (u >= STAGES) ok = mbar_wait(smem_u32(&ctrl->empty[u % STAGES]), ((u / STAGES) - 1) & 1, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            produce(u);
        }
        if (!ok && lane == 0 && p.status) atomicOr(p.status, 2u);
        return;
    }
    asm volatile("bar.sync 2, %0;" ::"n"(THREADS) : "memory");

    const int g = lane >> 2;  // mma row group; batch row of the B fragment
    const int t = lane & 3;
    // B fragments of this warp's 256-k slice: [group][limb][word][even|odd], and the per-(batch, group) step
    uint32_t xb[2][LIMBS][4][2];
    float dq[2][2];  // delta / 16 for the two batch columns (2t, 2t+1) of this lane's D fragment

    auto load_x = [&](uint32_t kb) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint4 v[4];
            float amax = 0.0f;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const uint32_t k0 = kb * KBLOCK + warp * WARP_K + c * 128 + t * 32 + wi * 8;
                v[wi] = make_uint4(0, 0, 0, 0);
                if (uint32_t(g) < p.m && k0 < p.k) v[wi] = *reinterpret_cast<const uint4*>(p.x + size_t(g) * p.k + k0);
                const uint32_t r[4] = {v[wi].x, v[wi].y, v[wi].z, v[wi].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(r[j])), fabsf(bf16_hi(r[j]))));
            }
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            // power-of-two step: |x| / delta < 2^(8*LIMBS - 1); exponent clamped so that 1/delta stays finite
            int e = int((__float_as_uint(amax) >> 23) & 0xFFu) - 127;
            e = max(e, -90);
            const int de = e - (8 * LIMBS - 2);                                   // delta = 2^de
            const float inv_delta = __uint_as_float(uint32_t(127 - de) << 23);    // 2^-de
            float delta16 = __uint_as_float(uint32_t(127 + de - 4) << 23);        // delta / 16
            if (e > 127) delta16 = __uint_as_float(0x7FC00000u);  // Inf/NaN activations poison their batch row
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const uint32_t r[4] = {v[wi].x, v[wi].y, v[wi].z, v[wi].w};
                int X[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    X[2 * j] = __float2int_rn(bf16_lo(r[j]) * inv_delta);
                    X[2 * j + 1] = __float2int_rn(bf16_hi(r[j]) * inv_delta);
                }
#pragma unroll
                for (int l = 0; l < LIMBS; ++l) {
                    // byte limb l of each element; the top limb keeps the sign through the arithmetic shift
                    auto limb = [&](int val) { return uint32_t(val >> (8 * l)) & 0xFFu; };
                    xb[c][l][wi][0] = limb(X[0]) | (limb(X[2]) << 8) | (limb(X[4]) << 16) | (limb(X[6]) << 24);
                    xb[c][l][wi][1] = limb(X[1]) | (limb(X[3]) << 8) | (limb(X[5]) << 16) | (limb(X[7]) << 24);
                }
            }
            // this lane's D fragment holds batch columns 2t and 2t+1: fetch their steps from lanes 4*(2t), 4*(2t+1)
            dq[c][0] = __shfl_sync(0xffffffffu, delta16, 4 * (2 * t));
            dq[c][1] = __shfl_sync(0xffffffffu, delta16, 4 * (2 * t + 1));
        }
    };
    // barrier over the 16 consumer warps only (the producer warp is busy feeding the ring)
    auto consumer_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(WARPS * 32) : "memory"); };
    if (coop) {
        uint8_t* xs = reinterpret_cast<uint8_t*>(red);                    // [LIMBS][m][X_PITCH] limb bytes
        float* dqs = reinterpret_cast<float*>(xs + stage_bytes_x);        // [m][32] delta / 16
        const uint32_t k0 = threadIdx.x * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (uint32_t(j) >= p.m) break;
            const uint32_t r[4] = {xv[j].x, xv[j].y, xv[j].z, xv[j].w};
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(r[i])), fabsf(bf16_hi(r[i]))));
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));  // 16 lanes = 1 group
            int e = int((__float_as_uint(amax) >> 23) & 0xFFu) - 127;
            e = max(e, -90);
            const int de = e - (8 * LIMBS - 2);
            const float inv_delta = __uint_as_float(uint32_t(127 - de) << 23);
            float delta16 = __uint_as_float(uint32_t(127 + de - 4) << 23);
            if (e > 127) delta16 = __uint_as_float(0x7FC00000u);
            int X[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if constexpr (LIMBS == 2) {
                    // |X| < 2^15: adding 1.5 * 2^23 leaves the rounded integer in the low mantissa bits
                    X[2 * i] = __float_as_int(fmaf(bf16_lo(r[i]), inv_delta, 12582912.0f)) - 0x4B400000;
                    X[2 * i + 1] = __float_as_int(fmaf(bf16_hi(r[i]), inv_delta, 12582912.0f)) - 0x4B400000;
                } else {
                    X[2 * i] = __float2int_rn(bf16_lo(r[i]) * inv_delta);
                    X[2 * i + 1] = __float2int_rn(bf16_hi(r[i]) * inv_delta);
                }
            }
#pragma unroll
            for (int l = 0; l < LIMBS; ++l) {
                auto limb = [&](int val) { return uint32_t(val >> (8 * l)) & 0xFFu; };
                uint2 pk;
                pk.x = limb(X[0]) | (limb(X[2]) << 8) | (limb(X[4]) << 16) | (limb(X[6]) << 24);
                pk.y = limb(X[1]) | (limb(X[3]) << 8) | (limb(X[5]) << 16) | (limb(X[7]) << 24);
                *reinterpret_cast<uint2*>(xs + (size_t(l) * p.m + j) * X_PITCH + k0) = pk;
            }
            if ((threadIdx.x & 15u) == 0) dqs[j * 32 + (threadIdx.x >> 4)] = delta16;
        }
        consumer_sync();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int l = 0; l < LIMBS; ++l) {
                uint4 a = make_uint4(0, 0, 0, 0), b = make_uint4(0, 0, 0, 0);
                if (uint32_t(g) < p.m) {
                    const uint8_t* src = xs + (size_t(l) * p.m + g) * X_PITCH + warp * WARP_K + c * 128 + t * 32;
                    a = *reinterpret_cast<const uint4*>(src);
                    b = *reinterpret_cast<const uint4*>(src + 16);
                }
                xb[c][l][0][0] = a.x; xb[c][l][0][1] = a.y; xb[c][l][1][0] = a.z; xb[c][l][1][1] = a.w;
                xb[c][l][2][0] = b.x; xb[c][l][2][1] = b.y; xb[c][l][3][0] = b.z; xb[c][l][3][1] = b.w;
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t col = 2 * t + j;
                dq[c][j] = col < p.m ? dqs[col * 32 + warp * 2 + c] : 0.0f;
            }
        }
        consumer_sync();  // the staging area is free again: it is the reduction slots from here on
    } else if (nkb == 1) {
        load_x(0);
    }

    // Register image of one 128-k group of this warp's slice: 16 B of each of the two fragment rows + 2 scales.
    // The loop below keeps one half in flight from shared memory while it does the math of the other.
    struct Half {
        uint4 wl, wh;
        uint32_t sc;  // bf16 scale of row g in the low half, of row g+8 in the high half
    };
    auto wait_full = [&](uint32_t u) -> bool {
        return mbar_wait(smem_u32(&ctrl->full[u % STAGES]), (u / STAGES) & 1, abort_flag);
    };
    auto load_half = [&](uint32_t u, int c, Half& h) {
        const uint8_t* stage = ring + size_t(u % STAGES) * STAGE_BYTES;
        const uint8_t* wrow = stage + g * row_pitch + warp * (WARP_K / 2) + c * 64 + t * 16;
        h.wl = *reinterpret_cast<const uint4*>(wrow);
        h.wh = *reinterpret_cast<const uint4*>(wrow + 8 * row_pitch);
        const uint8_t* srow = stage + STAGE_W_BYTES + g * scale_pitch + (warp * 2 + c) * 2;
        h.sc = uint32_t(*reinterpret_cast<const uint16_t*>(srow)) |
               (uint32_t(*reinterpret_cast<const uint16_t*>(srow + 8 * scale_pitch)) << 16);
    };
    auto release = [&](uint32_t u) {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->empty[u % STAGES]));
    };
    // one 128-k group: 4 words per row, two independent accumulator sets per limb (words 0-1 and 2-3)
    auto math_half = [&](const Half& h, const uint32_t (&xg)[LIMBS][4][2], const float (&dqg)[2], float (&out)[4]) {
        int acc[LIMBS][2][4];
#pragma unroll
        for (int l = 0; l < LIMBS; ++l)
#pragma unroll
            for (int q = 0; q < 2; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[l][q][i] = 0;
        const uint32_t lo[4] = {h.wl.x, h.wl.y, h.wl.z, h.wl.w};
        const uint32_t hi[4] = {h.wh.x, h.wh.y, h.wh.z, h.wh.w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            const uint32_t a0 = even_nibbles(lo[wi]), a1 = even_nibbles(hi[wi]);
            const uint32_t a2 = odd_nibbles(lo[wi]), a3 = odd_nibbles(hi[wi]);
#pragma unroll
            for (int l = 0; l < LIMBS; ++l) {
                if (l == LIMBS - 1)
                    mma_s8<true>(acc[l][wi >> 1], a0, a1, a2, a3, xg[l][wi][0], xg[l][wi][1]);
                else
                    mma_s8<false>(acc[l][wi >> 1], a0, a1, a2, a3, xg[l][wi][0], xg[l][wi][1]);
            }
        }
        const float s_lo = bf16_lo(h.sc), s_hi = bf16_hi(h.sc);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // every limb sum is below 2^24 in magnitude, so the int -> float conversions are exact
            float v = float(acc[LIMBS - 1][0][i] + acc[LIMBS - 1][1][i]);
#pragma unroll
            for (int l = LIMBS - 2; l >= 0; --l) v = fmaf(v, 256.0f, float(acc[l][0][i] + acc[l][1][i]));
            out[i] = fmaf((i < 2 ? s_lo : s_hi) * dqg[i & 1], v, out[i]);
        }
    };

    // sum the 16 partials of a finished tile and store its outputs (called by one designated warp per tile)
    auto reduce_tile = [&](uint32_t tile) -> bool {
        const uint32_t slot = tile % RED_SLOTS;
        bool ok = mbar_wait(smem_u32(&ctrl->red_full[slot]), (tile / RED_SLOTS) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return false;
        const float* slot_base = red + size_t(slot) * RED_SLOT_FLOATS;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float4 v = *reinterpret_cast<const float4*>(slot_base + w * 128 + lane * 4);
            sum.x += v.x;
            sum.y += v.y;
            sum.z += v.z;
            sum.w += v.w;
        }
        const uint32_t row_lo = r0 + tile * TILE_ROWS + g;
        const float vals[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t row = i < 2 ? row_lo : row_lo + 8;
            const uint32_t col = 2 * t + (i & 1);
            if (row < r1 && col < p.m) {
                if constexpr (OUT_F32)
                    static_cast<float*>(p.y)[size_t(col) * p.n + row] = vals[i];
                else
                    static_cast<__nv_bfloat16*>(p.y)[size_t(col) * p.n + row] = __float2bfloat16_rn(vals[i]);
            }
        }
        return true;
    };

    Half ha, hb;
    float out[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool alive = units == 0 || wait_full(0);
    if (alive && units > 0) load_half(0, 0, ha);
    for (uint32_t u = 0; u < units && alive; ++u) {
        const uint32_t tile = u / nkb, kb = u - tile * nkb;
        if (nkb != 1) load_x(kb);
        const bool active = kb * KBLOCK + warp * WARP_K < p.k;
        load_half(u, 1, hb);
        release(u);  // both halves of the unit have been read: the stage may be refilled while the math runs
        if (active) math_half(ha, xb[0], dq[0], out);
        if (u + 1 < units) {  // next unit's first half goes to registers behind the math of this unit's second
            alive = wait_full(u + 1);
            if (!alive) break;
            load_half(u + 1, 0, ha);
        }
        if (active) math_half(hb, xb[1], dq[1], out);
        if (kb + 1 == nkb) {
            // cross-warp reduction of the tile: every warp leaves its 16x8 partial in the tile's slot and arrives
            // on the slot barrier; warp (tile % 16) sums the slot one tile LATER, when the barrier has long
            // completed, so nobody waits. Partials are added in warp order: deterministic.
            const uint32_t slot = tile % RED_SLOTS;
            *reinterpret_cast<float4*>(red + size_t(slot) * RED_SLOT_FLOATS + warp * 128 + lane * 4) =
                make_float4(out[0], out[1], out[2], out[3]);
            out[0] = out[1] = out[2] = out[3] = 0.0f;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->red_full[slot]));
            if (tile > 0 && uint32_t(warp) == (tile - 1) % WARPS) alive = reduce_tile(tile - 1);
        }
    }
    if (alive && ntiles > 0 && uint32_t(warp) == (ntiles - 1) % WARPS) alive = reduce_tile(ntiles - 1);
    if (!alive && lane == 0 && p.status) atomicOr(p.status, 1u);
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

bool int4_gemv_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    return m >= 1 && m <= 8 && n >= 1 && group == 128 && k >= 1024 && k % 1024 == 0;
}

cudaError_t launch_int4_gemv(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                             uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                             uint32_t* status, bool constant_weights) {
    // Whole rows of 2048 or 4096 k: the half-SM kernel, whose launches overlap on every SM. bf16 outputs go four batch
    // rows at a time (26-bit block-floating activations, 57-bit for a single row); f32 outputs one row at a time, so
    // that every row gets the single-row precision.
    // Rows of 6144, 8192, ... (multiples of 2048 beyond 4096): the half-SM kernel per k block, sums carried in f32. bf16
    // outputs four batch rows at a time, f32 outputs one row at a time (single-row precision), like the whole-row path.
    if (int4_gemv_kblocks_supported(1, n, k, 128)) {
        const size_t out_elem = out_f32 ? 4 : 2;
        const uint32_t step = out_f32 ? 1 : 4;
        for (uint32_t b0 = 0; b0 < m; b0 += step) {
            const uint32_t mb = m - b0 < step ? m - b0 : step;
            cudaError_t e = launch_int4_gemv_kblocks(static_cast<const uint16_t*>(x_bf16) + size_t(b0) * k, w_packed, scale_bf16,
                                                     static_cast<uint8_t*>(y) + size_t(b0) * n * out_elem, mb, n, k, out_f32,
                                                     sm_count, stream, constant_weights);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    // Three to eight batch rows (f32 outputs: from two rows): one launch on the f16 tensor path, eight batch rows per MMA
    if (m >= (out_f32 ? 2u : 3u) && int4_gemv_batch8_supported(m, n, k, 128))
        return launch_int4_gemv_batch8(x_bf16, w_packed, scale_bf16, y, m, n, k, out_f32, sm_count, stream, constant_weights);
    if (int4_gemv_halfsm_supported(1, n, k, 128)) {
        const size_t out_elem = out_f32 ? 4 : 2;
        const uint32_t step = out_f32 ? 1 : 4;
        for (uint32_t b0 = 0; b0 < m; b0 += step) {
            const uint32_t mb = m - b0 < step ? m - b0 : step;
            cudaError_t e = launch_int4_gemv_halfsm(static_cast<const uint16_t*>(x_bf16) + size_t(b0) * k, w_packed, scale_bf16,
                                                    static_cast<uint8_t*>(y) + size_t(b0) * n * out_elem, mb, n, k, out_f32,
                                                    sm_count, stream, status, constant_weights);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    // opt in to the large dynamic shared-memory carve-out once per device
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t de = cudaGetDevice(&dev);
    if (de != cudaSuccess) return de;
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(int4_gemv_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_TOTAL);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(int4_gemv_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
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
    p.status = status;
    const uint32_t tiles = (n + TILE_ROWS - 1) / TILE_ROWS;
    const uint32_t grid = tiles < uint32_t(sm_count) ? tiles : uint32_t(sm_count);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    // with constant weights the launch may overlap the tail of the preceding kernel of the stream
    cfg.attrs = &attr;
    cfg.numAttrs = constant_weights ? 1 : 0;
    if (out_f32) return cudaLaunchKernelEx(&cfg, int4_gemv_kernel<4, true>, p);
    return cudaLaunchKernelEx(&cfg, int4_gemv_kernel<3, false>, p);
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

