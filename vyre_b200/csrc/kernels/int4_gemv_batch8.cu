// Decode GEMV for group-quantized int4 weights, batch 3..8 in ONE launch, k 2048 or 4096: the half-SM form on the
// f16 tensor path.
//
//   y[m, n] = cast( sum_k x[m, k] * (q[n, k] - 8) * s[n, k / 128] )
//
// Same launch shape as int4_gemv_halfsm.cu (one CTA per SM that takes less than half an SM, so that under programmatic
// dependent launch the next launch's CTA sits beside it with its first three tiles of weights on their way; per-warp
// three-stage cp.async pipelines over 16-row tiles; no barrier between warps in the stream). What differs is the math.
// The integer path of that kernel spends four of the eight B columns of an MMA on the digits of ONE batch row, so four
// batch rows cost twice the MMAs and eight rows a second launch that reads the weights again. Here the eight B columns
// are eight batch rows:
//
//  * mma.sync.m16n8k16, f16 x f16 -> f32. A = 16 weight rows, B = this warp's k slice of up to eight batch rows, held
//    in registers for the whole kernel (64 registers at k = 4096).
//  * Weights become f16 without a lookup and with one shift per eight: a nibble n that sits in bits [3:0] of a 16-bit
//    half is 1024 + n under exponent pattern 0x6400, one in bits [7:4] is 64 + n under 0x5400; `w` and `w >> 8` hold all
//    eight nibbles of a word in those two positions. One f16x2 subtraction (1032 or 72, exact) gives q - 8. The k labels
//    inside an MMA are a dummy index, so the pairing of nibbles (i, i + 4) in one register is matched by pairing the
//    activations the same way when they are loaded.
//  * Activations: bf16 -> f16 per (batch row, 128-k group) after an exact power-of-two scaling that puts the group's
//    largest magnitude into [2^14, 2^15). f16 has 11 significant bits (bf16: 8), so every element down to 2^-29 of its
//    group's largest is represented exactly (and smaller ones to 2^-39 of it); the products are exact in f32 and a
//    zero weight contributes exactly zero. The scaling is undone in the f32 factor the group's sum is multiplied by
//    together with the weight scale. Inf / NaN activations poison their group's outputs.
//  * No smem scratch, no cross-lane sums: the MMA sums over k inside the warp; per tile a warp leaves a 16 x 8 partial
//    in its own corner of shared memory, and after three tiles (what that corner holds) one barrier and a fixed-order
//    sum over the warps (deterministic).
//
// Nothing in the kernel waits on a flag or an mbarrier: it cannot hang.
//
// Replaces the generated scalar kernel of vyre-libs/src/nn/linear/inner/linear_4bit.rs:399-775 (one warp per output)
// for the row-major layout of vyre-primitives/src/math/quantized/programs.rs:186-300 at decode batches.
#include <cuda_bf16.h>

#include <atomic>

#include "kernels.h"

namespace vybk {
namespace {

constexpr int TILE_ROWS = 16;
constexpr int STAGES = 3;
constexpr int NB = 8;                                          // batch rows = B columns of the MMA
constexpr int SMEM_W = STAGES * TILE_ROWS * 2048;              // weight stages of all warps: 3 tiles of 16 rows x 4096 k
constexpr int SMEM_S = STAGES * TILE_ROWS * 64;                // their scales
constexpr int SMEM_RED = 12288;                                // per-warp partial sums
constexpr int SMEM_TOTAL = SMEM_W + SMEM_S + SMEM_RED;
constexpr uint32_t PACE_NS = 400;

static_assert(2 * (SMEM_TOTAL + 1024) <= 233472, "two CTAs must fit one SM");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sub_f16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// {high half: hi, low half: lo} as f16, round to nearest even
__device__ __forceinline__ uint32_t pack_f16x2(float hi, float lo) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
// nibbles in bits [3:0] of both halves -> q - 8 as f16x2; the same for bits [7:4]
__device__ __forceinline__ uint32_t nib_lo(uint32_t w) { return sub_f16x2((w & 0x000F000Fu) | 0x64006400u, 0x64086408u); }
__device__ __forceinline__ uint32_t nib_hi(uint32_t w) { return sub_f16x2((w & 0x00F000F0u) | 0x54005400u, 0x54805480u); }
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

struct Params {
    const uint16_t* x;
    const uint8_t* w;
    const uint16_t* scales;
    void* y;
    uint32_t m, n;
    uint32_t tiles_per_cta, tiles_rem;  // whole 16-row tiles per CTA; the first tiles_rem CTAs own one more
    uint32_t pace_ns;                   // pause between the prefetched tiles (0: none)
};

// W warps, each owning GPW 128-k groups of every row: k = 128 GPW W
template <int GPW, int W, bool OUT_F32>
__global__ void __launch_bounds__(W * 32, 2) int4_gemv_batch8_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    // let the next launch of the stream become resident beside this one at once; it waits (griddepcontrol.wait)
    // before it reads activations or writes outputs. A no-op for plain launches.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr uint32_t K = 128u * GPW * W;
    constexpr uint32_t ROW_BYTES = K / 2;            // packed bytes of one row of W
    constexpr uint32_t PITCH = GPW * 64;             // of which this warp owns (= row pitch of its stages)
    constexpr uint32_t CPR = GPW * 4;                // 16-byte chunks per row slice
    constexpr uint32_t RPI = 32 / CPR;               // rows covered by one warp-wide cp.async
    constexpr uint32_t NCP = TILE_ROWS / RPI;        // cp.async instructions per tile and lane
    constexpr uint32_t WSTAGE = TILE_ROWS * PITCH;   // bytes of one warp's share of a tile
    constexpr uint32_t SSTAGE = TILE_ROWS * GPW * 2; // and of its scales
    constexpr uint32_t PART = TILE_ROWS * NB * 4;    // bytes of one warp's partial of one tile
    constexpr uint32_t PRIV = SMEM_RED / W;          // bytes of partials a warp owns
    constexpr uint32_t FLUSH = PRIV / PART;          // tiles between two reductions
    static_assert(FLUSH >= 1, "a warp's area must hold a tile's partial");
    static_assert(GPW == 2 || GPW == 4, "a warp owns 256 or 512 k");
    static_assert(RPI % 2 == 0, "the row parity of a lane must not depend on the copy index");
    static_assert(W * STAGES * (WSTAGE + SSTAGE) <= SMEM_W + SMEM_S, "stages must fit");

    uint8_t* red = smem + SMEM_W + SMEM_S;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t first_tile = blockIdx.x * p.tiles_per_cta + min(blockIdx.x, p.tiles_rem);
    const uint32_t r0 = first_tile * TILE_ROWS;
    const uint32_t r1 = min(p.n, r0 + (p.tiles_per_cta + (blockIdx.x < p.tiles_rem ? 1u : 0u)) * TILE_ROWS);
    const uint32_t nrows = r1 - r0;
    const uint32_t ntiles = (nrows + TILE_ROWS - 1) / TILE_ROWS;
    uint8_t* my_w = smem + warp * (STAGES * WSTAGE);             // this warp's private weight stages
    uint8_t* my_s = smem + SMEM_W + warp * (STAGES * SSTAGE);    // and their scales

    // ---- this warp's private weight pipeline: one commit group per tile, STAGES tiles deep ---------------------
    // Lane l of copy i moves chunk l % CPR of row i * RPI + l / CPR. Odd rows are stored with the two 64-byte halves of
    // every 128 bytes swapped: a 128-bit fragment load is served a quarter warp at a time (rows 2q and 2q+1, four
    // consecutive chunks each), and the swap puts those eight chunks into eight different 16-byte bank groups.
    const uint32_t cp_row = lane / CPR, cp_chunk = lane % CPR;
    const uint8_t* cp_src = p.w + size_t(r0 + cp_row) * ROW_BYTES + warp * PITCH + cp_chunk * 16;
    const uint32_t cp_dst = smem_u32(my_w) + cp_row * PITCH + ((cp_chunk ^ ((cp_row & 1u) << 2)) << 4);
    const uint32_t sc_row = lane / (GPW / 2), sc_unit = lane % (GPW / 2);  // 4-byte units of scales
    const uint16_t* sc_src = p.scales + size_t(r0 + sc_row) * (K / 128) + warp * GPW + sc_unit * 2;
    const uint32_t sc_dst = smem_u32(my_s) + sc_row * (GPW * 2) + sc_unit * 4;
    uint32_t issue_stage = 0, issue_rows = nrows;  // stage offset index and rows left for the next tile to issue
    auto issue_tile = [&]() {
        if (issue_rows > 0) {
            const uint32_t dst = cp_dst + issue_stage * WSTAGE;
            if (issue_rows >= TILE_ROWS) {  // every tile but possibly the last
#pragma unroll
                for (uint32_t i = 0; i < NCP; ++i) cp_async_16(dst + i * RPI * PITCH, cp_src + i * RPI * ROW_BYTES);
                if (GPW == 4 || sc_row < TILE_ROWS) cp_async_4(sc_dst + issue_stage * SSTAGE, sc_src);
            } else {
#pragma unroll
                for (uint32_t i = 0; i < NCP; ++i)
                    if (cp_row + i * RPI < issue_rows) cp_async_16(dst + i * RPI * PITCH, cp_src + i * RPI * ROW_BYTES);
                if (sc_row < issue_rows) cp_async_4(sc_dst + issue_stage * SSTAGE, sc_src);
            }
            cp_src += TILE_ROWS * ROW_BYTES;
            sc_src += TILE_ROWS * (K / 128);
            issue_rows = issue_rows > TILE_ROWS ? issue_rows - TILE_ROWS : 0u;
            issue_stage = issue_stage == STAGES - 1 ? 0u : issue_stage + 1;
        }
        cp_async_commit();
    };
    // Weights are constants: prefetched before the dependency wait, paced so that the predecessor's activation loads on
    // the same SM do not queue behind a 96 KB burst.
#pragma unroll
    for (int u = 0; u < STAGES; ++u) {
        if (u > 0 && p.pace_ns) __nanosleep(p.pace_ns);
        issue_tile();
    }

    const uint32_t g = lane >> 2;  // A/D fragment row, B fragment column (= batch row)
    const uint32_t t = lane & 3;

    // ---- activations: everything below reads x, so the previous launch of the stream must be complete ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // This lane's B fragments: batch row g, k = 128 c + 32 t + 8 u + (0..7) of the warp's slice, i.e. the elements under
    // the lane's 16-byte weight chunk 4c + t. Word u of that chunk feeds two MMAs: nibbles (0,4) and (1,5), then (2,6)
    // and (3,7); the activations are paired the same way.
    uint32_t xb[GPW][4][4];
    float dq[GPW][2];  // 2^-shift of (batch rows 2t and 2t+1, group): the D columns of this lane
#pragma unroll
    for (int c = 0; c < GPW; ++c) {
        // group by group: a burst of all the slice's loads at once measured slower (it competes with the prefetch of the
        // next launch's CTA on the same SM)
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) raw[u] = make_uint4(0, 0, 0, 0);
        if (g < p.m) {
            const uint4* src = reinterpret_cast<const uint4*>(p.x + size_t(g) * K + warp * (GPW * 128) + c * 128 + t * 32);
#pragma unroll
            for (int u = 0; u < 4; ++u) raw[u] = __ldcg(src + u);
        }
        // largest magnitude of the group as an integer maximum of |bits| (a NaN orders above infinity)
        uint32_t amax = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t r[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) amax = max(amax, max((r[i] << 16) & 0x7FFF0000u, r[i] & 0x7FFF0000u));
        }
        amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, 2));  // the four lanes of a batch row hold its group
        const int ebits = int(amax >> 23);  // biased exponent; 255 = Inf or NaN in the group
        const int e = max(ebits - 127, -100);
        const float up = __uint_as_float(uint32_t(127 + 14 - e) << 23);  // 2^(14 - e): the largest lands in [2^14, 2^15)
        float down = __uint_as_float(uint32_t(127 + e - 14) << 23);
        if (ebits == 255) down = __uint_as_float(0x7FC00000u);  // Inf/NaN activations poison their group's outputs
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t r[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};  // r[i] = elements 2i (low half), 2i + 1
            xb[c][u][0] = pack_f16x2(bf16_lo(r[2]) * up, bf16_lo(r[0]) * up);  // elements (0, 4)
            xb[c][u][1] = pack_f16x2(bf16_hi(r[2]) * up, bf16_hi(r[0]) * up);  // (1, 5)
            xb[c][u][2] = pack_f16x2(bf16_lo(r[3]) * up, bf16_lo(r[1]) * up);  // (2, 6)
            xb[c][u][3] = pack_f16x2(bf16_hi(r[3]) * up, bf16_hi(r[1]) * up);  // (3, 7)
        }
        dq[c][0] = __shfl_sync(0xffffffffu, down, 8 * t);
        dq[c][1] = __shfl_sync(0xffffffffu, down, 8 * t + 4);
    }

    // sum the warps' partials of the tiles [first, first + count) in warp order and store the outputs
    auto reduce_tiles = [&](uint32_t first, uint32_t count) {
        __syncthreads();
        for (uint32_t idx = threadIdx.x; idx < count * (TILE_ROWS * NB); idx += W * 32) {
            // [tile][col][row] order of the threads: neighbouring threads store neighbouring outputs
            const uint32_t tile = idx / (TILE_ROWS * NB), col = (idx / TILE_ROWS) % NB, rr = idx % TILE_ROWS;
            const uint32_t row = r0 + (first + tile) * TILE_ROWS + rr;
            const float* src = reinterpret_cast<const float*>(red) + tile * (PART / 4) + rr * NB + col;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < W; ++w) sum += src[w * (PRIV / 4)];
            if (row < r1 && col < p.m) {
                if constexpr (OUT_F32) static_cast<float*>(p.y)[size_t(col) * p.n + row] = sum;
                else static_cast<__nv_bfloat16*>(p.y)[size_t(col) * p.n + row] = __float2bfloat16_rn(sum);
            }
        }
    };

    // fragment addresses inside a stage: chunk 4c + t of row g (and g + 8), halves swapped in odd rows
    const uint32_t lds_base = g * PITCH + (t << 4);
    const uint32_t lds_even = lds_base + ((g & 1u) << 6);         // group 0 (and 2: +128)
    const uint32_t lds_odd = lds_base + (((g & 1u) ^ 1u) << 6);   // group 1 (and 3: +128)
    const uint32_t lds_scale = g * (GPW * 2);

    uint32_t stage = 0, pending = 0;  // pending: tiles whose partials wait in shared memory
    float* part = reinterpret_cast<float*>(red + warp * PRIV) + g * NB + 2 * t;
    for (uint32_t u = 0; u < ntiles; ++u) {
        cp_async_wait<STAGES - 1>();  // this thread's copies of tile u have landed ...
        __syncwarp();                 // ... and so have the other lanes'
        const uint8_t* ws = my_w + stage * WSTAGE;
        const uint8_t* ss = my_s + stage * SSTAGE + lds_scale;
        stage = stage == STAGES - 1 ? 0u : stage + 1;
        // bf16 scales of this warp's groups: row g in sa, row g + 8 in sb
        uint32_t sa[GPW / 2], sb[GPW / 2];
        if constexpr (GPW == 4) {
            const uint2 a = *reinterpret_cast<const uint2*>(ss);
            const uint2 b = *reinterpret_cast<const uint2*>(ss + 8 * GPW * 2);
            sa[0] = a.x; sa[1] = a.y; sb[0] = b.x; sb[1] = b.y;
        } else {
            sa[0] = *reinterpret_cast<const uint32_t*>(ss);
            sb[0] = *reinterpret_cast<const uint32_t*>(ss + 8 * GPW * 2);
        }
        float P[4] = {0.f, 0.f, 0.f, 0.f};  // (row g, batch 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
#pragma unroll
        for (int h = 0; h < GPW / 2; ++h) {
            // two groups at a time in registers; once the last pair is read the stage is refilled under the math
            uint4 wl[2], wh[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int c = 2 * h + i;
                const uint8_t* src = ws + ((c & 1) ? lds_odd : lds_even) + (c >> 1) * 128;
                wl[i] = *reinterpret_cast<const uint4*>(src);
                wh[i] = *reinterpret_cast<const uint4*>(src + 8 * PITCH);
            }
            if (h == GPW / 2 - 1) {
                __syncwarp();
                issue_tile();
            }
            float acc[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
            const uint32_t lo[2][4] = {{wl[0].x, wl[0].y, wl[0].z, wl[0].w}, {wl[1].x, wl[1].y, wl[1].z, wl[1].w}};
            const uint32_t hi[2][4] = {{wh[0].x, wh[0].y, wh[0].z, wh[0].w}, {wh[1].x, wh[1].y, wh[1].z, wh[1].w}};
#pragma unroll
            for (int uu = 0; uu < 4; ++uu) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {  // the two groups' chains interleave
                    const int c = 2 * h + i;
                    const uint32_t w0 = lo[i][uu], w1 = hi[i][uu];
                    mma_f16(acc[i], nib_lo(w0), nib_lo(w1), nib_hi(w0), nib_hi(w1), xb[c][uu][0], xb[c][uu][1]);
                    const uint32_t v0 = w0 >> 8, v1 = w1 >> 8;
                    mma_f16(acc[i], nib_lo(v0), nib_lo(v1), nib_hi(v0), nib_hi(v1), xb[c][uu][2], xb[c][uu][3]);
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int c = 2 * h + i;
                const float s_lo = (c & 1) ? bf16_hi(sa[c >> 1]) : bf16_lo(sa[c >> 1]);
                const float s_hi = (c & 1) ? bf16_hi(sb[c >> 1]) : bf16_lo(sb[c >> 1]);
                P[0] = fmaf(s_lo * dq[c][0], acc[i][0], P[0]);
                P[1] = fmaf(s_lo * dq[c][1], acc[i][1], P[1]);
                P[2] = fmaf(s_hi * dq[c][0], acc[i][2], P[2]);
                P[3] = fmaf(s_hi * dq[c][1], acc[i][3], P[3]);
            }
        }
        *reinterpret_cast<float2*>(part + pending * (PART / 4)) = make_float2(P[0], P[1]);
        *reinterpret_cast<float2*>(part + pending * (PART / 4) + 8 * NB) = make_float2(P[2], P[3]);
        ++pending;
        if (pending == FLUSH && u + 1 < ntiles) {  // the warp's corner is full: sum what has piled up and start over
            reduce_tiles(u + 1 - FLUSH, FLUSH);
            __syncthreads();
            pending = 0;
        }
    }
    cp_async_wait<0>();
    if (pending) reduce_tiles(ntiles - pending, pending);
}

}  // namespace

bool int4_gemv_batch8_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    return m >= 1 && m <= 8 && n >= 1 && group == 128 && (k == 2048 || k == 4096);
}

cudaError_t launch_int4_gemv_batch8(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                    uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                                    bool constant_weights) {
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t de = cudaGetDevice(&dev);
    if (de != cudaSuccess) return de;
    const uint64_t bit = 1ull << (dev & 63);
    using Kernel = void (*)(const Params);
    static const Kernel kernels[2][2] = {{int4_gemv_batch8_kernel<4, 8, false>, int4_gemv_batch8_kernel<4, 8, true>},
                                         {int4_gemv_batch8_kernel<2, 8, false>, int4_gemv_batch8_kernel<2, 8, true>}};
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        for (int i = 0; i < 4; ++i) {
            const void* f = (const void*)kernels[i / 2][i % 2];
            cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (e != cudaSuccess) return e;
        }
        configured.fetch_or(bit, std::memory_order_release);
    }
    Params p;
    p.x = static_cast<const uint16_t*>(x_bf16);
    p.w = static_cast<const uint8_t*>(w_packed);
    p.scales = static_cast<const uint16_t*>(scale_bf16);
    p.y = y;
    p.m = m;
    p.n = n;
    p.pace_ns = constant_weights ? PACE_NS : 0u;
    // one CTA per SM, whole 16-row tiles each, the remainder spread one tile per CTA
    const uint32_t tiles = (n + TILE_ROWS - 1) / TILE_ROWS;
    const uint32_t grid = tiles < uint32_t(sm_count) ? tiles : uint32_t(sm_count);
    p.tiles_per_cta = tiles / grid;
    p.tiles_rem = tiles % grid;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = SMEM_TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = constant_weights ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernels[k == 4096 ? 0 : 1][out_f32 ? 1 : 0], p);
}

}  // namespace vybk
