// Decode GEMV for group-quantized int4 weights, batch <= 4, k <= 4096: the half-SM form.
//
//   y[m, n] = cast( sum_k x[m, k] * (q[n, k] - 8) * s[n, k / 128] )
//
// A decode GEMV moves about 200 KB of weights per SM and launch, a few microseconds of HBM time, so what a
// launch costs beyond its bytes (start-up, the first loads' latency, the last tile's reduction, the gap to the
// next launch) weighs as much as the stream itself. This kernel is shaped so that consecutive launches of a
// stream overlap on every SM:
//
//  * One CTA per SM and launch, and that CTA takes LESS THAN HALF of an SM: 512 threads at <= 64 registers (batch
//    <= 2, k = 4096) or 256 threads at <= 128 registers, and 113 KB of shared memory. With programmatic dependent launch the next launch's CTA becomes resident beside
//    this one, prefetches three tiles of (constant) weights and only then waits for this launch to finish before
//    it touches activations or outputs. While launch N works through the tail of its rows, launch N+1's weights
//    are already on their way, so HBM does not idle at a launch boundary. The trigger
//    (griddepcontrol.launch_dependents) is the first instruction of the kernel.
//  * Each warp owns a fixed slice of k (256 or 512 wide) and runs its OWN three-deep pipeline over the 16-row tiles:
//    16-byte cp.async copies (the load/store path, which streams finer-grained than 32 KB bulk copies: a warp
//    refills its few KB as soon as it has read them) into a private region of shared memory, completion by
//    cp.async.wait_group, no barrier between warps anywhere in the stream. Rows are stored with their 16-byte
//    chunks XOR-swizzled by the row number so that the fragment loads of eight rows hit eight bank groups.
//  * Math runs on the integer tensor path (mma.sync.m16n8k32, u8 x s8 -> s32) with ONE logic instruction per eight
//    weights. A packed byte b = 16 q1 + q0 holds the weights of elements 2j and 2j+1. With integer activations
//    X0, X1:  b * (16 X0) + (b & 0xF0) * (X1 - 16 X0) = 16 (q0 X0 + q1 X1). So the raw bytes are one A operand as
//    they are, the masked bytes (`w & 0xF0F0F0F0`) the other, and the two B operands (16 X0 and X1 - 16 X0) are
//    prepared once per CTA. The zero point costs nothing per weight either: sum 16 (q - 8) X = sum 16 q X -
//    128 sum X, and -128 sum X (per group, known once the activations are converted) is what the group's
//    accumulators start from.
//  * Activations are converted once per CTA to block-floating integers: per (batch row, 128-k group) a power-of-two
//    step delta = 2^(e_max - 25) and X = rint(x / delta), |X| < 2^26; the B values above stay below 2^31 and are
//    written as four balanced base-256 digits d0..d3 in [-128, 127]. bf16 carries 8 significant bits, so every
//    element within 2^-18 of its group's largest is represented EXACTLY; a smaller one is rounded to 2^-26 of the
//    group maximum. The four digits of a batch row occupy four of the eight B-operand columns of the MMA (two batch
//    rows per MMA). A single batch row has all eight columns: a warp whose slice holds an element below that 2^-18
//    converts it with eight digits (|X| < 2^57, exact down to 2^-49 of the largest); the stream is not touched, but that launch's prologue takes about 1 us longer (measured 7.3 against 6.2 us at 28672 x 2048; about 3 % of N(0,1) rows of 4096 hold such an element). The integer sums are exact; per group the digit sums are recombined (d0 + 256 d1 in integers,
//    the 65536 between digit pairs folded into the f32 factor) and scaled by s * delta / 16 in f32, the only place
//    rounding happens.
//  * The activation fragments of a warp's k slice stay in registers for the whole kernel, so shared memory is
//    read once per weight byte. Per tile each warp leaves a 16 x batch partial in its own corner of shared
//    memory; after the last tile (or every few tiles, when a CTA owns many) one barrier, and every thread sums the
//    warps' partials of one output in fixed order (deterministic).
//
//  * FUSED instantiations take the neighbours of a residual block into the launch: a learned RMSNorm of the activations in
//    the prologue (one CTA barrier for the row's sum of squares), SwiGLU with another projection's outputs as the gate or a
//    residual add where a finished sum is rounded and stored; every intermediate is rounded as the stand-alone operators
//    round it, so the outputs are those of the operators run one after the other.
//
// Nothing in the kernel waits on another warp except those barriers, and nothing waits on a flag or an mbarrier: it
// cannot hang.
//
// Replaces the generated scalar kernel of vyre-libs/src/nn/linear/inner/linear_4bit.rs:399-775 (one warp per
// output, 4-byte loads, scalar f32 FMA) for the row-major layout of
// vyre-primitives/src/math/quantized/programs.rs:186-300.
#include <cuda_bf16.h>

#include <atomic>
#include <map>
#include <mutex>
#include <utility>

#include "kernels.h"
#include "peer_gather.cuh"

namespace vybk {
namespace {

constexpr int TILE_ROWS = 16;
constexpr int STAGES = 3;
constexpr int SMEM_W = STAGES * TILE_ROWS * 2048;             // weight stages of all warps: 3 tiles of 16 rows x 4096 k
constexpr int SMEM_S = STAGES * TILE_ROWS * 64;               // their scales
constexpr int SMEM_RED = 12288;                               // per-warp partial sums; the activation scratch of the prologue
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
// D(16x8, s32) = A(16x32, u8, row) * B(32x8, s8, col) + C
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, int c0, int c1, int c2, int c3) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}
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
    // the gathering form only: the outputs go to this rank's slice of buffer half `half` on EVERY rank
    PeerGather ag;
    uint32_t half;
    uint32_t pipelined;  // the peer stores of launch d are issued at the start of launch d + 1 and drain under its work
    uint32_t* status;
    // the k-block form only (STRIDED): this launch covers K columns of a wider matrix
    uint32_t row_bytes;     // packed bytes between two rows of W
    uint32_t scale_stride;  // scales between two rows
    uint32_t x_stride;      // elements between two batch rows of x
    const float* acc_in;    // [m][n] f32 sums of the k blocks before this one (nullptr: none), added in the reduction
    // one launch over all k blocks (kblocks > 1): CTA i works on k block i % kblocks, leaves f32 partial rows in `part` and
    // counts an arrival per 16-row tile; the CTA whose arrival completes a tile sums its kblocks partials in block order
    uint32_t kblocks;
    float* part;            // [kblocks][m][n]
    uint32_t* tile_count;   // [tiles], zero between launches (the last arriver resets its word)
    // the residual block around the projection (FUSED instantiations; the k-block form honours `resid` and `gate` as well): a learned
    // RMSNorm of the activations in the prologue and a residual add in the output stores, with the roundings of the
    // stand-alone operators (normalised value to bf16, times weight to bf16; sum to bf16, plus residual to bf16)
    const uint16_t* norm_w;  // [k] bf16 (nullptr: no norm)
    float norm_eps;
    const uint16_t* resid;   // [m][n] bf16 (nullptr: no residual add)
    // SwiGLU behind an up projection: gate holds the gate projection's outputs ([m][n] bf16); the stores write
    // gate * (up * sigmoid(gate)) with up = this launch's sums rounded to bf16 (nullptr: none; not together with resid)
    const uint16_t* gate;
};

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }
// The stand-alone SwiGLU's arithmetic (vyre-libs/src/nn/activation/unary.rs:79-100: gate * (up * (1 / (1 + exp(-gate)))), every
// f32 operation rounded to nearest with subnormals flushed, one cast to bf16) on this launch's sum as `up`, rounded to bf16
// first as the stand-alone projection stores it. Out of line: a handful of outputs per thread, off the main loop's registers.
__device__ __forceinline__ float mul_ftz(float a, float b) {
    float r;
    asm("mul.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float add_ftz(float a, float b) {
    float r;
    asm("add.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float div_ftz(float a, float b) {
    float r;
    asm("div.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __noinline__ __nv_bfloat16 swiglu_of(const uint16_t* gate, size_t at, float sum) {
    const float g = bf16_bits_to_float(__ldcg(gate + at)), u = __bfloat162float(__float2bfloat16_rn(sum));
    const float sig = div_ftz(1.0f, add_ftz(1.0f, expf(-g)));
    return __float2bfloat16_rn(mul_ftz(g, mul_ftz(u, sig)));
}
// cast(bf16, f32(residual) + f32(branch)) with the branch already rounded to bf16 (vyre-libs/src/nn/activation/residual_add.rs:40-52)
__device__ __forceinline__ __nv_bfloat16 add_residual(const uint16_t* resid, size_t at, float sum) {
    return __float2bfloat16_rn(__fadd_rn(bf16_bits_to_float(__ldcg(resid + at)), __bfloat162float(__float2bfloat16_rn(sum))));
}

// k split inside one launch: count this CTA's arrival for the tiles [tile0, tile0 + count); where it is the last of the
// k blocks to arrive, sum the partial rows in block order (deterministic) and store the outputs. Out of line.
template <bool OUT_F32>
__device__ __noinline__ void ksplit_finish(const Params& p, uint32_t tile0, uint32_t count, uint32_t* flags) {
    __syncthreads();  // the CTA's partial stores are ordered before the fences below; the shared-memory partials are consumed
    if (threadIdx.x < count) {
        __threadfence();  // cumulative: publishes the whole CTA's partial rows before the arrival
        uint32_t* word = p.tile_count + tile0 + threadIdx.x;
        const bool last = atomicAdd(word, 1u) == p.kblocks - 1;
        if (last) {
            *word = 0u;       // nobody else touches the word until the next launch
            __threadfence();  // the other blocks' partial rows, published before their arrivals, are visible from here on
        }
        flags[threadIdx.x] = last ? 1u : 0u;
    }
    __syncthreads();
    const uint32_t per_tile = 16 * p.m;
    for (uint32_t idx = threadIdx.x; idx < count * per_tile; idx += blockDim.x) {
        const uint32_t t = idx / per_tile, rem = idx % per_tile;
        if (!flags[t]) continue;
        const uint32_t col = rem / 16, row = (tile0 + t) * 16 + rem % 16;
        if (row >= p.n) continue;
        // all loads first (independent, one L2 round trip), then the sum in block order
        const float* src = p.part + size_t(col) * p.n + row;
        const size_t stride = size_t(p.m) * p.n;
        float v[16];
#pragma unroll
        for (uint32_t b = 0; b < 16; ++b) v[b] = b < p.kblocks ? __ldcg(src + b * stride) : 0.f;
        float sum = 0.f;
#pragma unroll
        for (uint32_t b = 0; b < 16; ++b) sum += v[b];
        for (uint32_t b = 16; b < p.kblocks; ++b) sum += __ldcg(src + b * stride);
        const size_t at = size_t(col) * p.n + row;
        if (OUT_F32) static_cast<float*>(p.y)[at] = sum;
        else
            static_cast<__nv_bfloat16*>(p.y)[at] = p.gate    ? swiglu_of(p.gate, at, sum)
                                                   : p.resid ? add_residual(p.resid, at, sum)
                                                             : __float2bfloat16_rn(sum);
    }
    __syncthreads();
}

// Pipelined gathering form, kept out of line (the kernel below runs at the edge of its register budget): carry the
// predecessor's slice, which sits in the other buffer half of local memory, to the peers. The stores drain under this
// launch's tiles. The peers are past whatever consumed the slice this one replaces when they have signalled two launches
// back (a signal sent a whole launch ago, so this does not wait in a healthy run). Bounded; status bit 128.
__device__ __noinline__ void gather_carry(const Params& p, uint32_t r0, uint32_t nrows) {
    const uint32_t lane = threadIdx.x & 31;
    volatile uint32_t* e = reinterpret_cast<volatile uint32_t*>(p.ag.epoch);
    const uint32_t pending = e[EPOCH_PUSH];
    uint32_t pushed = 0;
    if (pending == (p.half ^ 1u) + 1 && p.ag.world > 1) {  // halves alternate: the slice left by the launch before
        const uint32_t index = e[EPOCH_INDEX + p.half];
        if (lane < p.ag.world && lane != p.ag.rank && index >= 2 && !wait_pushes_from(p.ag, lane, index - 2, p.status) && p.status)
            atomicOr(p.status, 128u);
        __syncwarp();
        const size_t base = (size_t(pending - 1) * p.ag.world + p.ag.rank) * p.m * p.n;
        const uint16_t* src = reinterpret_cast<const uint16_t*>(p.ag.peer_out[p.ag.rank]) + base;
        for (uint32_t i = threadIdx.x; i < nrows * p.m; i += blockDim.x) {
            const size_t at = size_t(i / nrows) * p.n + r0 + i % nrows;
            const uint16_t v = __ldcg(src + at);
            for (uint32_t q = 0; q < p.ag.world; ++q)
                if (q != p.ag.rank) reinterpret_cast<uint16_t*>(p.ag.peer_out[q])[base + at] = v;
        }
        pushed = 1;
    }
    // what this launch carries over is complete when the launch ends: the signal for it is owed to the next launch
    if (blockIdx.x == 0 && threadIdx.x == 0) e[EPOCH_OWED] = pushed;
}

// NM = MMAs per 16 rows x 32 k = ceil(m / 2); W warps, each owning GPW 128-k groups of every row: k = 128 GPW W
// GATHER: a column-parallel shard whose bf16 outputs are stored straight into every rank's gather buffer (peer stores over
// NVLink from the reduction that produces them), so that the all-gather is part of the launch and consecutive launches
// stay one programmatic chain. No CTA fences at system scope: the arrival signal of launch d is sent by whatever runs
// next on the stream (launch d + 1 or the wait kernel), when launch d is complete and its stores are visible. Before it
// stores into a peer's half, a launch checks (bounded) that this peer has signalled launch d - 1: then the peer is past
// whatever consumed launch d - 2 from the same half. Buffer halves must alternate from launch to launch.
// Pipelined form (Params::pipelined): a launch cannot end before its peer stores have drained (an NVLink round trip), and
// the next launch's activations wait for exactly that. So launch d stores into the LOCAL buffer only and leaves its slice
// to launch d + 1, whose CTAs copy their own rows of it to the peers right after the dependency wait (gather_carry). The
// arrival signal for slice d is then sent by launch d + 2, or by the wait kernel, which also carries the last slice over.
template <int NM, int GPW, int W, bool OUT_F32, bool GATHER, bool STRIDED = false, bool FUSED = false>
__global__ void __launch_bounds__(W * 32, 2) int4_gemv_halfsm_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    // let the next launch of the stream become resident beside this one at once; it waits (griddepcontrol.wait)
    // before it reads activations or writes outputs. A no-op for plain launches.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr uint32_t K = 128u * GPW * W;
    constexpr uint32_t ROW_BYTES_DENSE = K / 2;      // packed bytes of one row of W when the launch covers whole rows
    constexpr uint32_t PITCH = GPW * 64;             // of which this warp owns (= row pitch of its stages)
    constexpr uint32_t CPR = GPW * 4;                // 16-byte chunks per row slice
    constexpr uint32_t RPI = 32 / CPR;               // rows covered by one warp-wide cp.async
    constexpr uint32_t NCP = TILE_ROWS / RPI;        // cp.async instructions per tile and lane
    constexpr uint32_t WSTAGE = TILE_ROWS * PITCH;   // bytes of one warp's share of a tile
    constexpr uint32_t SSTAGE = TILE_ROWS * GPW * 2; // and of its scales
    constexpr uint32_t MM = 2 * NM;                  // batch rows of a partial
    constexpr uint32_t PART = TILE_ROWS * MM * 4;    // bytes of one warp's partial of one tile
    // A warp's tile of a 2048-k row is half as large. Whole rows of 2048: six stages instead of three keep as many bytes in
    // flight per CTA (6.9 -> 6.2 us at 28672 rows). The k-block form keeps three stages and puts its partial sums into the
    // unused upper half of the weight stages, so that four times as many tiles fit between two reductions: there every
    // reduction ends in the arrival protocol of the k split, and six stages with a reduction every 12 tiles measured
    // slower (4096 x 14336: 12.1 us against 9.3 us).
    constexpr bool DEEP = GPW == 2 && !STRIDED;
    constexpr int ST = DEEP ? 2 * STAGES : STAGES;
    constexpr uint32_t RED_BYTES = (GPW == 4 || DEEP) ? SMEM_RED : SMEM_W / 2;
    constexpr uint32_t PRIV = RED_BYTES / W;         // bytes of partials (and prologue scratch) a warp owns
    constexpr uint32_t FLUSH = PRIV / PART;          // tiles between two reductions
    static_assert(PRIV >= 2 * GPW * 128, "the activation scratch must fit a warp's own area");
    static_assert(GPW == 2 || GPW == 4, "a warp owns 256 or 512 k");
    static_assert(RPI % 2 == 0, "the row parity of a lane must not depend on the copy index");
    static_assert(W * ST * (WSTAGE + SSTAGE) <= SMEM_W + SMEM_S, "stages must fit");

    uint8_t* red = smem + ((GPW == 4 || DEEP) ? SMEM_W + SMEM_S : SMEM_W / 2);
    // whole rows: compile-time strides; a k block of a wider matrix (STRIDED): the strides of that matrix
    const uint32_t ROW_BYTES = STRIDED ? p.row_bytes : ROW_BYTES_DENSE;
    const uint32_t SCALE_STRIDE = STRIDED ? p.scale_stride : K / 128;
    const uint32_t X_STRIDE = STRIDED ? p.x_stride : K;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    // whole tiles per CTA, the first tiles_rem CTAs one more than the rest
    uint32_t first_tile = blockIdx.x * p.tiles_per_cta + min(blockIdx.x, p.tiles_rem);
    uint32_t my_tiles = p.tiles_per_cta + (blockIdx.x < p.tiles_rem ? 1u : 0u);
    uint32_t kblock = 0;  // STRIDED with kblocks > 1: the k block of this CTA; its tiles are split among the CTAs of that block
    if constexpr (STRIDED) {
        if (p.kblocks > 1) {
            kblock = blockIdx.x % p.kblocks;
            const uint32_t gi = blockIdx.x / p.kblocks, gn = (gridDim.x - kblock + p.kblocks - 1) / p.kblocks;
            const uint32_t total = (p.n + TILE_ROWS - 1) / TILE_ROWS, per = total / gn, extra = total % gn;
            first_tile = gi * per + min(gi, extra);
            my_tiles = per + (gi < extra ? 1u : 0u);
        }
    }
    const uint32_t r0 = first_tile * TILE_ROWS;
    const uint32_t r1 = min(p.n, r0 + my_tiles * TILE_ROWS);
    const uint32_t nrows = r1 - r0;
    const uint32_t ntiles = (nrows + TILE_ROWS - 1) / TILE_ROWS;
    uint8_t* my_w = smem + warp * (ST * WSTAGE);             // this warp's private weight stages
    uint8_t* my_s = smem + SMEM_W + warp * (ST * SSTAGE);    // and their scales

    // ---- this warp's private weight pipeline: one commit group per tile, STAGES tiles deep ---------------------
    // Lane l of copy i moves chunk l % CPR of row i * RPI + l / CPR. Odd rows are stored with the two 64-byte halves of
    // every 128 bytes swapped: a 128-bit fragment load is served a quarter warp at a time (rows 2q and 2q+1, four
    // consecutive chunks each), and the swap puts those eight chunks into eight different 16-byte bank groups.
    const uint32_t cp_row = lane / CPR, cp_chunk = lane % CPR;
    const uint8_t* cp_src = p.w + size_t(r0 + cp_row) * ROW_BYTES + kblock * (K / 2) + warp * PITCH + cp_chunk * 16;
    const uint32_t cp_dst = smem_u32(my_w) + cp_row * PITCH + ((cp_chunk ^ ((cp_row & 1u) << 2)) << 4);
    const uint32_t sc_row = lane / (GPW / 2), sc_unit = lane % (GPW / 2);  // 4-byte units of scales
    const uint16_t* sc_src = p.scales + size_t(r0 + sc_row) * SCALE_STRIDE + kblock * (K / 128) + warp * GPW + sc_unit * 2;
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
            sc_src += TILE_ROWS * SCALE_STRIDE;
            issue_rows = issue_rows > TILE_ROWS ? issue_rows - TILE_ROWS : 0u;
            issue_stage = issue_stage == ST - 1 ? 0u : issue_stage + 1;
        }
        cp_async_commit();
    };
    // Weights are constants: prefetched before the dependency wait. Under programmatic dependent launch this CTA arrives
    // on its SM just when its predecessor is about to be released and load its activations through the same load/store
    // queue, so the prefetch is paced (about PACE_NS between tiles) rather than issued as one 96 KB burst that the
    // predecessor's few activation loads would have to queue behind. This CTA has microseconds to spare here.
#pragma unroll
    for (int u = 0; u < ST; ++u) {
        if (u > 0 && p.pace_ns) __nanosleep(DEEP ? p.pace_ns / 2 : p.pace_ns);  // the same bytes per pause
        issue_tile();
    }

    const uint32_t g = lane >> 2;  // A/D fragment row, B fragment column
    const uint32_t t = lane & 3;

    // ---- activations: everything below reads x, so the previous launch of the stream must be complete ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t launch_index = 0;  // GATHER: how many gathering launches this rank has completed before this one
    if constexpr (GATHER) {
        launch_index = *(reinterpret_cast<const volatile uint32_t*>(p.ag.epoch) + EPOCH_INDEX + p.half);
        if (blockIdx.x == 0 && warp == 0) send_owed_signal(p.ag, lane);  // the previous launch's arrival
        if (p.pipelined) gather_carry(p, r0, nrows);
    }
    // FUSED with a norm weight: 1 / sqrt(mean(x^2) + eps) of every batch row, the sum of squares in the order of the
    // stand-alone operator's long-row form (thread t adds elements t, t + 256, ...; a butterfly over the warp; the eight
    // warp sums in warp order), so that the fused launch gives the bits of norm-then-projection
    float inv_rms[2 * NM];
    uint4 pre_x[2 * NM][2], pre_w[2];  // FUSED with a norm weight: this lane's 16 activations of every row and their weights,
                                       // loaded ahead so that their round trip overlaps the one of the sum's loads
    if constexpr (FUSED) {
        static_assert(W == 8 && !GATHER && !STRIDED && !OUT_F32, "the fused block is the dense bf16 form of 256 threads");
        __shared__ float warp_sq[2 * NM][W];
#pragma unroll
        for (int j = 0; j < 2 * NM; ++j) inv_rms[j] = 0.0f;
        if (p.norm_w) {
            const bool mine = lane < GPW * 8;  // 16 elements per lane cover the warp's slice
#pragma unroll
            for (int j = 0; j < 2 * NM; ++j) {
                pre_x[j][0] = pre_x[j][1] = make_uint4(0, 0, 0, 0);
                if (uint32_t(j) < p.m && mine) {
                    const uint4* src = reinterpret_cast<const uint4*>(p.x + size_t(j) * K + warp * (GPW * 128) + lane * 16);
                    pre_x[j][0] = __ldcg(src);
                    pre_x[j][1] = __ldcg(src + 1);
                }
            }
            pre_w[0] = pre_w[1] = make_uint4(0, 0, 0, 0);
            if (mine) {
                const uint4* wsrc = reinterpret_cast<const uint4*>(p.norm_w + warp * (GPW * 128) + lane * 16);
                pre_w[0] = __ldg(wsrc);
                pre_w[1] = __ldg(wsrc + 1);
            }
#pragma unroll
            for (int j = 0; j < 2 * NM; ++j) {
                if (uint32_t(j) >= p.m) break;
                const uint16_t* row = p.x + size_t(j) * K;
                uint16_t own[K / (W * 32)];  // all loads in flight at once, then the sum in index order
#pragma unroll
                for (uint32_t i = 0; i < K / (W * 32); ++i) own[i] = __ldcg(row + threadIdx.x + i * (W * 32));
                float sum = 0.0f;
#pragma unroll
                for (uint32_t i = 0; i < K / (W * 32); ++i) {
                    const float v = bf16_bits_to_float(own[i]);
                    sum = __fadd_rn(sum, __fmul_rn(v, v));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
                if (lane == 0) warp_sq[j][warp] = sum;
            }
            __syncthreads();
#pragma unroll
            for (int j = 0; j < 2 * NM; ++j) {
                if (uint32_t(j) >= p.m) break;
                float total = 0.0f;
#pragma unroll
                for (int w = 0; w < W; ++w) total = __fadd_rn(total, warp_sq[j][w]);
                inv_rms[j] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, float(K)), p.norm_eps)));
            }
        }
    }
    uint32_t xb[NM][GPW][8];  // [mma][group of this warp][byte block 0 | 1][operand 0 | 1][bytes 0-3 | 4-7]
    float dq[NM][GPW];        // delta / 16 of (batch row of this lane's D columns, group), x 65536 for the high digit pair
    int corr[NM][GPW];        // -128 x (sum of the group's X, low or high 16-bit part) for this lane's D columns: zero point
#pragma unroll
    for (int nm = 0; nm < NM; ++nm)
#pragma unroll
        for (int c = 0; c < GPW; ++c) {
            dq[nm][c] = 0.0f;
            corr[nm][c] = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) xb[nm][c][i] = 0u;
        }
    {
        // Every warp converts its OWN k slice (16 elements per lane) and hands the digits to the lanes that need them
        // through scratch that only this warp touches: its own area of partial sums, which nobody else reads before the
        // first reduction barrier. No CTA barrier.
        constexpr uint32_t DIGIT_BYTES = GPW * 128;  // one digit of the slice: 8 bytes of each operand per 16 elements
        auto scratch = [&](uint32_t off) -> uint8_t* { return red + warp * PRIV + off; };
        const bool has = lane < GPW * 8;  // 16 elements per lane cover the slice
#pragma unroll
        for (int j = 0; j < 2 * NM; ++j) {
            if (uint32_t(j) >= p.m) break;
            uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
            bool preloaded = false;
            if constexpr (FUSED) {
                if (p.norm_w) {
                    x0 = pre_x[j][0];
                    x1 = pre_x[j][1];
                    preloaded = true;
                }
            }
            if (has && !preloaded) {
                const uint4* src = reinterpret_cast<const uint4*>(p.x + size_t(j) * X_STRIDE + kblock * K + warp * (GPW * 128) + lane * 16);
                x0 = __ldcg(src);
                x1 = __ldcg(src + 1);
            }
            uint32_t r[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};  // r[i] = elements 2i (low half), 2i+1
            if constexpr (FUSED) {
                if (p.norm_w && has) {  // x * inv to bf16, times the weight to bf16: the stand-alone operator's two roundings
                    const uint4 g0 = pre_w[0], g1 = pre_w[1];
                    const uint32_t gw[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                    auto norm1 = [&](float x, float w) -> uint32_t {
                        const float n = __bfloat162float(__float2bfloat16_rn(__fmul_rn(x, inv_rms[j])));
                        return uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(n, w))));
                    };
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        r[i] = norm1(bf16_lo(r[i]), bf16_lo(gw[i])) | (norm1(bf16_hi(r[i]), bf16_hi(gw[i])) << 16);
                }
            }
            // largest magnitude of the group as an integer maximum of |bits| (positive floats order like their bits, and a
            // NaN, which a float maximum would drop, orders above infinity)
            uint32_t amax = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = max(amax, max((r[i] << 16) & 0x7FFF0000u, r[i] & 0x7FFF0000u));
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, o));  // 8 lanes = 1 group
            const int ebits = int(amax >> 23);  // biased exponent; 255 = Inf or NaN in the group
            const int e = max(ebits - 127, -90);
            const int de = e - 25;                                              // delta = 2^de, |x / delta| < 2^26
            const float inv_delta = __uint_as_float(uint32_t(127 - de) << 23);  // 2^-de
            float delta16 = __uint_as_float(uint32_t(127 + de - 4) << 23);      // delta / 16
            if (ebits == 255) delta16 = __uint_as_float(0x7FC00000u);  // Inf/NaN activations poison their group's outputs
            // per packed byte i (elements 2i, 2i+1): operand 0 = 16 X0, operand 1 = X1 - 16 X0, each as four balanced
            // base-256 digits at once: with Y = V + 0x808080 the low three bytes of Y, top bit flipped, are d0..d2 in
            // [-128, 127] and the top byte of Y is d3. Also the sums of the low and high 16-bit parts of X.
            uint32_t z0[8], z1[8];
            int sum_lo = 0, sum_hi = 0;
            bool small = false;  // some nonzero element was rounded: |x / delta| < 2^7 cannot hold its 8 significant bits
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int X0 = __float2int_rn(bf16_lo(r[i]) * inv_delta), X1 = __float2int_rn(bf16_hi(r[i]) * inv_delta);
                if (NM == 1) small |= ((r[i] & 0x7FFFu) != 0 && abs(X0) < 128) | ((r[i] & 0x7FFF0000u) != 0 && abs(X1) < 128);
                const int V0 = X0 << 4, V1 = X1 - V0;
                z0[i] = uint32_t(V0 + 0x00808080) ^ 0x00808080u;
                z1[i] = uint32_t(V1 + 0x00808080) ^ 0x00808080u;
                const int Y0 = X0 + 0x8000, Y1 = X1 + 0x8000;  // X = (Y >> 16) * 65536 + ((Y & 0xFFFF) - 0x8000)
                sum_hi += (Y0 >> 16) + (Y1 >> 16);
                sum_lo += int(Y0 & 0xFFFF) + int(Y1 & 0xFFFF) - 0x10000;
            }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, o);
                sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, o);
            }
            if constexpr (NM == 1) {
                // A single batch row has all eight B columns to itself. When some element of this warp's slice lies more
                // than 2^18 below its group's largest (four digits have just rounded it: a nonzero bf16 whose integer
                // image has fewer than its 8 significant bits), the slice is converted again with eight digits:
                // |X| < 2^57, exact for every element within 2^-49 of the largest.
                if (p.m == 1) {
                    if (__any_sync(0xffffffffu, small)) {
                        const int ew = max(ebits - 127, -60);
                        float delta16 = __uint_as_float(uint32_t(127 + ew - 60) << 23);  // delta / 16, delta = 2^(ew - 56)
                        if (ebits == 255) delta16 = __uint_as_float(0x7FC00000u);
                        uint32_t zl[2][8], zh[2][8];  // [operand][byte]: digits 0-3 and 4-7 of its value
                        int psum[4] = {0, 0, 0, 0};   // sums of the four balanced 16-bit parts of X
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            long long X[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const uint32_t b = h ? (r[i] >> 16) : (r[i] & 0xFFFFu);
                                const int eb = int((b >> 7) & 0xFFu);
                                const long long m8 = eb ? (long long)((b & 0x7Fu) | 0x80u) : 0ll;  // x = m8 * 2^(eb - 134)
                                const int sh = eb - ew - 78;                                        // X = m8 * 2^sh
                                long long v = sh >= 0 ? (m8 << min(sh, 50)) : (sh > -10 ? ((m8 + (1ll << (-sh - 1))) >> -sh) : 0ll);
                                X[h] = (b & 0x8000u) ? -v : v;
                                const long long Y = X[h] + 0x0000800080008000ll;
                                psum[0] += int(Y & 0xFFFF) - 0x8000;
                                psum[1] += int((Y >> 16) & 0xFFFF) - 0x8000;
                                psum[2] += int((Y >> 32) & 0xFFFF) - 0x8000;
                                psum[3] += int(Y >> 48);
                            }
                            const long long V0 = X[0] << 4, V1 = X[1] - V0;
                            const unsigned long long Z0 = (unsigned long long)(V0 + 0x0080808080808080ll) ^ 0x0080808080808080ull;
                            const unsigned long long Z1 = (unsigned long long)(V1 + 0x0080808080808080ll) ^ 0x0080808080808080ull;
                            zl[0][i] = uint32_t(Z0); zh[0][i] = uint32_t(Z0 >> 32);
                            zl[1][i] = uint32_t(Z1); zh[1][i] = uint32_t(Z1 >> 32);
                        }
#pragma unroll
                        for (int d = 0; d < 4; ++d)
#pragma unroll
                            for (int o = 1; o < 8; o <<= 1) psum[d] += __shfl_xor_sync(0xffffffffu, psum[d], o);
                        uint32_t dig8[8][4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                const uint32_t* z = half ? zh[q >> 1] : zl[q >> 1];
                                const int b = (q & 1) * 4;
                                const uint32_t t0 = __byte_perm(z[b], z[b + 1], 0x5140), t1 = __byte_perm(z[b], z[b + 1], 0x7362);
                                const uint32_t t2 = __byte_perm(z[b + 2], z[b + 3], 0x5140), t3 = __byte_perm(z[b + 2], z[b + 3], 0x7362);
                                dig8[4 * half + 0][q] = __byte_perm(t0, t2, 0x5410);
                                dig8[4 * half + 1][q] = __byte_perm(t0, t2, 0x7632);
                                dig8[4 * half + 2][q] = __byte_perm(t1, t3, 0x5410);
                                dig8[4 * half + 3][q] = __byte_perm(t1, t3, 0x7632);
                            }
                        }
#pragma unroll
                        for (int ph = 0; ph < 4; ++ph) {
                            if (has) {
                                *reinterpret_cast<uint4*>(scratch(lane * 16)) =
                                    make_uint4(dig8[2 * ph][0], dig8[2 * ph][1], dig8[2 * ph][2], dig8[2 * ph][3]);
                                *reinterpret_cast<uint4*>(scratch(DIGIT_BYTES + lane * 16)) =
                                    make_uint4(dig8[2 * ph + 1][0], dig8[2 * ph + 1][1], dig8[2 * ph + 1][2], dig8[2 * ph + 1][3]);
                            }
                            __syncwarp();
                            if ((g >> 1) == uint32_t(ph)) {  // B column g holds digit g
#pragma unroll
                                for (int c = 0; c < GPW; ++c) {
                                    const uint8_t* src = scratch((g & 1) * DIGIT_BYTES + c * 128) + t * 32;
                                    const uint4 a = *reinterpret_cast<const uint4*>(src);
                                    const uint4 b = *reinterpret_cast<const uint4*>(src + 16);
                                    uint32_t(&dst)[8] = xb[0][c];
                                    dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
                                    dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
                                }
                            }
                            __syncwarp();
                        }
                        // D columns 2t, 2t+1 hold digits 2t, 2t+1: the 16-bit part t of X, weight 65536^t
#pragma unroll
                        for (int c = 0; c < GPW; ++c) {
                            const float d = __shfl_sync(0xffffffffu, delta16, c * 8);
                            int sp[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) sp[q] = __shfl_sync(0xffffffffu, psum[q], c * 8);
                            dq[0][c] = d * __uint_as_float((127u + 16u * t) << 23);
                            corr[0][c] = (t == 0 ? sp[0] : t == 1 ? sp[1] : t == 2 ? sp[2] : sp[3]) * -128;
                        }
                        break;
                    }
                }
            }
            // byte transpose: dig[d] = digit d of (operand 0 bytes 0-3, operand 0 bytes 4-7, operand 1 bytes 0-3, 4-7)
            uint32_t dig[4][4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t* z = (q & 2) ? z1 : z0;
                const int b = (q & 1) * 4;
                const uint32_t t0 = __byte_perm(z[b], z[b + 1], 0x5140), t1 = __byte_perm(z[b], z[b + 1], 0x7362);
                const uint32_t t2 = __byte_perm(z[b + 2], z[b + 3], 0x5140), t3 = __byte_perm(z[b + 2], z[b + 3], 0x7362);
                dig[0][q] = __byte_perm(t0, t2, 0x5410);
                dig[1][q] = __byte_perm(t0, t2, 0x7632);
                dig[2][q] = __byte_perm(t1, t3, 0x5410);
                dig[3][q] = __byte_perm(t1, t3, 0x7632);
            }
#pragma unroll
            for (int ph = 0; ph < 2; ++ph) {
                if (has) {
                    *reinterpret_cast<uint4*>(scratch(lane * 16)) = make_uint4(dig[2 * ph][0], dig[2 * ph][1], dig[2 * ph][2], dig[2 * ph][3]);
                    *reinterpret_cast<uint4*>(scratch(DIGIT_BYTES + lane * 16)) =
                        make_uint4(dig[2 * ph + 1][0], dig[2 * ph + 1][1], dig[2 * ph + 1][2], dig[2 * ph + 1][3]);
                }
                __syncwarp();
                // B column g holds digit g % 4 of batch row 2 nm + g / 4; this lane's 16 weight bytes of group c were
                // converted by lanes 8c + 2t (byte block 0) and 8c + 2t + 1 (byte block 1)
                if ((g >> 2) == uint32_t(j & 1) && ((g >> 1) & 1) == uint32_t(ph)) {
#pragma unroll
                    for (int c = 0; c < GPW; ++c) {
                        const uint8_t* src = scratch((g & 1) * DIGIT_BYTES + c * 128) + t * 32;
                        const uint4 a = *reinterpret_cast<const uint4*>(src);
                        const uint4 b = *reinterpret_cast<const uint4*>(src + 16);
                        uint32_t(&dst)[8] = xb[j >> 1][c];
                        dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
                        dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
                    }
                }
                __syncwarp();
            }
            // D columns 2t, 2t+1 hold digits 2 (t & 1), +1 of batch row 2 nm + t / 2; group c was converted by lanes 8c..
#pragma unroll
            for (int c = 0; c < GPW; ++c) {
                const float d = __shfl_sync(0xffffffffu, delta16, c * 8);
                const int sl = __shfl_sync(0xffffffffu, sum_lo, c * 8), sh = __shfl_sync(0xffffffffu, sum_hi, c * 8);
                if ((t >> 1) == uint32_t(j & 1)) {
                    dq[j >> 1][c] = d * ((t & 1) ? 65536.0f : 1.0f);
                    corr[j >> 1][c] = ((t & 1) ? sh : sl) * -128;
                }
            }
        }
    }

    // sum the warps' partials of the tiles [first, first + count) in warp order and store the outputs
    bool peers_checked = false;
    auto reduce_tiles = [&](uint32_t first, uint32_t count) {
        if constexpr (GATHER) {
            // every peer has signalled its launch before this one (sent when this launch began over there, microseconds
            // ago): its consumers of the half about to be overwritten have run. Bounded; status bit 128 when it runs out.
            if (!peers_checked && !p.pipelined && warp == 0 && lane < p.ag.world && lane != p.ag.rank &&
                !wait_pushes_from(p.ag, lane, launch_index, p.status) && p.status)
                atomicOr(p.status, 128u);
            peers_checked = true;
        }
        __syncthreads();
        for (uint32_t idx = threadIdx.x; idx < count * (TILE_ROWS * MM); idx += W * 32) {
            const uint32_t col = idx % MM, row = r0 + first * TILE_ROWS + idx / MM;
            const float* src = reinterpret_cast<const float*>(red) + idx;  // [tile][row][col] inside a warp's area
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < W; ++w) sum += src[w * (PRIV / 4)];
            if constexpr (STRIDED) {
                if (p.acc_in && row < r1 && col < p.m) sum += p.acc_in[size_t(col) * p.n + row];
                if (p.kblocks > 1) {  // one launch over all k blocks: this block's partial row
                    if (row < r1 && col < p.m) p.part[(size_t(kblock) * p.m + col) * p.n + row] = sum;
                    continue;
                }
            }
            if (row < r1 && col < p.m) {
                if constexpr (GATHER) {
                    const size_t at = (size_t(p.half) * p.ag.world + p.ag.rank) * p.m * p.n + size_t(col) * p.n + row;
                    const __nv_bfloat16 v = __float2bfloat16_rn(sum);
                    // plain form: every rank's buffer; pipelined form: this rank's only (the next launch carries it over)
                    const uint32_t q0 = p.pipelined ? p.ag.rank : 0u, q1 = p.pipelined ? p.ag.rank + 1 : p.ag.world;
                    for (uint32_t q = q0; q < q1; ++q) reinterpret_cast<__nv_bfloat16*>(p.ag.peer_out[q])[at] = v;
                } else if constexpr (OUT_F32) {
                    static_cast<float*>(p.y)[size_t(col) * p.n + row] = sum;
                } else if constexpr (FUSED) {
                    const size_t at = size_t(col) * p.n + row;
                    static_cast<__nv_bfloat16*>(p.y)[at] = p.gate    ? swiglu_of(p.gate, at, sum)
                                                           : p.resid ? add_residual(p.resid, at, sum)
                                                                     : __float2bfloat16_rn(sum);
                } else {
                    static_cast<__nv_bfloat16*>(p.y)[size_t(col) * p.n + row] = __float2bfloat16_rn(sum);
                }
            }
        }
        if constexpr (STRIDED) {
            if (p.kblocks > 1) ksplit_finish<OUT_F32>(p, first_tile + first, count, reinterpret_cast<uint32_t*>(red));
        }
    };

    // fragment addresses inside a stage: chunk 4c + t of row g (and g + 8), halves swapped in odd rows
    const uint32_t lds_base = g * PITCH + (t << 4);
    const uint32_t lds_even = lds_base + ((g & 1u) << 6);         // group 0 (and 2: +128)
    const uint32_t lds_odd = lds_base + (((g & 1u) ^ 1u) << 6);   // group 1 (and 3: +128)
    const uint32_t lds_scale = g * (GPW * 2);

    uint32_t stage = 0, pending = 0;  // pending: tiles whose partials wait in shared memory
    float* part = reinterpret_cast<float*>(red + warp * PRIV) + g * MM + (t >> 1);
    float Pq[NM][2];                  // the previous tile's per-lane partials, not yet summed across lanes
    bool have_q = false;
    // low and high digit pairs of a batch row sit in neighbouring lanes; a single batch row may use all four pairs
    auto fold_partials = [&]() {
        if (!have_q) return;
        have_q = false;
#pragma unroll
        for (int nm = 0; nm < NM; ++nm) {
            Pq[nm][0] += __shfl_xor_sync(0xffffffffu, Pq[nm][0], 1);
            Pq[nm][1] += __shfl_xor_sync(0xffffffffu, Pq[nm][1], 1);
        }
        if (NM == 1 && p.m == 1) {
            Pq[0][0] += __shfl_xor_sync(0xffffffffu, Pq[0][0], 2);
            Pq[0][1] += __shfl_xor_sync(0xffffffffu, Pq[0][1], 2);
        }
        if ((t & 1) == 0 && !(NM == 1 && p.m == 1 && t != 0)) {
#pragma unroll
            for (int nm = 0; nm < NM; ++nm) {
                part[pending * (PART / 4) + 2 * nm] = Pq[nm][0];
                part[pending * (PART / 4) + 8 * MM + 2 * nm] = Pq[nm][1];
            }
        }
        ++pending;
    };
    for (uint32_t u = 0; u < ntiles; ++u) {
        cp_async_wait<ST - 1>();  // this thread's copies of tile u have landed ...
        __syncwarp();                 // ... and so have the other lanes'
        const uint8_t* ws = my_w + stage * WSTAGE;
        const uint8_t* ss = my_s + stage * SSTAGE + lds_scale;
        stage = stage == ST - 1 ? 0u : stage + 1;
        uint4 wl[GPW], wh[GPW];
#pragma unroll
        for (int c = 0; c < GPW; ++c) {
            const uint8_t* src = ws + ((c & 1) ? lds_odd : lds_even) + (c >> 1) * 128;
            wl[c] = *reinterpret_cast<const uint4*>(src);
            wh[c] = *reinterpret_cast<const uint4*>(src + 8 * PITCH);
        }
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
        // the whole slice of the tile sits in registers: refill the stage while the math runs
        __syncwarp();
        issue_tile();
        fold_partials();  // of the previous tile

        float P[NM][2];
#pragma unroll
        for (int nm = 0; nm < NM; ++nm) P[nm][0] = P[nm][1] = 0.0f;
        if constexpr (NM == 1) {
            // The four MMAs of a group form a dependent chain (about 25 cycles each), so the groups are interleaved: every
            // step issues one MMA of each group, and a group's next MMA finds its accumulators ready.
            int acc[GPW][NM][4];
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                // raw bytes against 16 X0 ...
#pragma unroll
                for (int c = 0; c < GPW; ++c) {
                    const uint32_t a0 = blk ? wl[c].z : wl[c].x, a1 = blk ? wh[c].z : wh[c].x;
                    const uint32_t a2 = blk ? wl[c].w : wl[c].y, a3 = blk ? wh[c].w : wh[c].y;
#pragma unroll
                    for (int nm = 0; nm < NM; ++nm) {
                        if (blk == 0)  // the group's accumulators start from the zero-point term (all of it in the low digit)
                            mma_u8s8(acc[c][nm], a0, a1, a2, a3, xb[nm][c][0], xb[nm][c][1], corr[nm][c], 0, corr[nm][c], 0);
                        else
                            mma_u8s8(acc[c][nm], a0, a1, a2, a3, xb[nm][c][4], xb[nm][c][5], acc[c][nm][0], acc[c][nm][1],
                                     acc[c][nm][2], acc[c][nm][3]);
                    }
                }
                // ... then masked bytes against X1 - 16 X0
#pragma unroll
                for (int c = 0; c < GPW; ++c) {
                    const uint32_t m0 = (blk ? wl[c].z : wl[c].x) & 0xF0F0F0F0u, m1 = (blk ? wh[c].z : wh[c].x) & 0xF0F0F0F0u;
                    const uint32_t m2 = (blk ? wl[c].w : wl[c].y) & 0xF0F0F0F0u, m3 = (blk ? wh[c].w : wh[c].y) & 0xF0F0F0F0u;
#pragma unroll
                    for (int nm = 0; nm < NM; ++nm)
                        mma_u8s8(acc[c][nm], m0, m1, m2, m3, xb[nm][c][4 * blk + 2], xb[nm][c][4 * blk + 3], acc[c][nm][0],
                                 acc[c][nm][1], acc[c][nm][2], acc[c][nm][3]);
                }
            }
#pragma unroll
            for (int c = 0; c < GPW; ++c) {
                const float s_lo = (c & 1) ? bf16_hi(sa[c >> 1]) : bf16_lo(sa[c >> 1]);
                const float s_hi = (c & 1) ? bf16_hi(sb[c >> 1]) : bf16_lo(sb[c >> 1]);
#pragma unroll
                for (int nm = 0; nm < NM; ++nm) {
                    // |accumulators| < 2^22 per group and |zero-point term| < 2^29: d_lo + 256 d_hi stays below 2^31
                    const float v_lo = float(acc[c][nm][0] + (acc[c][nm][1] << 8));
                    const float v_hi = float(acc[c][nm][2] + (acc[c][nm][3] << 8));
                    P[nm][0] = fmaf(s_lo * dq[nm][c], v_lo, P[nm][0]);
                    P[nm][1] = fmaf(s_hi * dq[nm][c], v_hi, P[nm][1]);
                }
            }
        } else {  // two MMAs per step already overlap; interleaving the groups as well costs registers this variant lacks
#pragma unroll
            for (int c = 0; c < GPW; ++c) {
                int acc[NM][4];
                const uint32_t lo[4] = {wl[c].x, wl[c].y, wl[c].z, wl[c].w};
                const uint32_t hi[4] = {wh[c].x, wh[c].y, wh[c].z, wh[c].w};
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    // raw bytes against 16 X0, then masked bytes against X1 - 16 X0
                    const uint32_t a0 = lo[2 * blk], a1 = hi[2 * blk], a2 = lo[2 * blk + 1], a3 = hi[2 * blk + 1];
                    const uint32_t m0 = a0 & 0xF0F0F0F0u, m1 = a1 & 0xF0F0F0F0u, m2 = a2 & 0xF0F0F0F0u, m3 = a3 & 0xF0F0F0F0u;
#pragma unroll
                    for (int nm = 0; nm < NM; ++nm) {
                        if (blk == 0)  // the group's accumulators start from the zero-point term (all of it in the low digit)
                            mma_u8s8(acc[nm], a0, a1, a2, a3, xb[nm][c][0], xb[nm][c][1], corr[nm][c], 0, corr[nm][c], 0);
                        else
                            mma_u8s8(acc[nm], a0, a1, a2, a3, xb[nm][c][4], xb[nm][c][5], acc[nm][0], acc[nm][1], acc[nm][2], acc[nm][3]);
                        mma_u8s8(acc[nm], m0, m1, m2, m3, xb[nm][c][4 * blk + 2], xb[nm][c][4 * blk + 3], acc[nm][0], acc[nm][1],
                                 acc[nm][2], acc[nm][3]);
                    }
                }
                const float s_lo = (c & 1) ? bf16_hi(sa[c >> 1]) : bf16_lo(sa[c >> 1]);
                const float s_hi = (c & 1) ? bf16_hi(sb[c >> 1]) : bf16_lo(sb[c >> 1]);
#pragma unroll
                for (int nm = 0; nm < NM; ++nm) {
                    // |accumulators| < 2^22 per group and |zero-point term| < 2^29: d_lo + 256 d_hi stays below 2^31
                    const float v_lo = float(acc[nm][0] + (acc[nm][1] << 8));
                    const float v_hi = float(acc[nm][2] + (acc[nm][3] << 8));
                    P[nm][0] = fmaf(s_lo * dq[nm][c], v_lo, P[nm][0]);
                    P[nm][1] = fmaf(s_hi * dq[nm][c], v_hi, P[nm][1]);
                }
            }
        }
        // The cross-lane sum of this tile's partials (shuffles, each waiting for the one before) is left for the next
        // iteration, where it runs under the latency of that tile's shared-memory loads.
#pragma unroll
        for (int nm = 0; nm < NM; ++nm) {
            Pq[nm][0] = P[nm][0];
            Pq[nm][1] = P[nm][1];
        }
        have_q = true;
        if (pending + 1 == FLUSH && u + 1 < ntiles) {  // a CTA with many tiles: sum what has piled up and start over
            fold_partials();
            reduce_tiles(u + 1 - FLUSH, FLUSH);
            __syncthreads();
            pending = 0;
        }
    }
    fold_partials();
    cp_async_wait<0>();
    if (pending) reduce_tiles(ntiles - pending, pending);
    if constexpr (GATHER) {
        // one CTA hands the launch index to the next launch (which reads the other half's word), counts the launch for the
        // wait kernel and leaves the arrival signal owed
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            volatile uint32_t* e = reinterpret_cast<volatile uint32_t*>(p.ag.epoch);
            e[EPOCH_INDEX + (p.half ^ 1u)] = launch_index + 1;
            for (uint32_t i = 0; i + 1 < p.ag.world || i == 0; ++i) e[i] = launch_index + 1;
            if (p.pipelined) {
                e[EPOCH_PUSH] = p.half + 1;  // this launch's slice waits in local memory
                e[EPOCH_PUSH_M] = p.m;
                e[EPOCH_PUSH_N] = p.n;
            } else {
                e[EPOCH_OWED] = 1;
            }
        }
    }
}

}  // namespace

bool int4_gemv_halfsm_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    return m >= 1 && m <= 4 && n >= 1 && group == 128 && (k == 2048 || k == 4096);
}

cudaError_t launch_int4_gemv_halfsm(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                    uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                                    uint32_t* status, bool constant_weights, const PeerGather* gather, uint32_t half, bool pipelined,
                                    const void* norm_w, float norm_eps, const void* resid, const void* gate) {
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t de = cudaGetDevice(&dev);
    if (de != cudaSuccess) return de;
    const uint64_t bit = 1ull << (dev & 63);
    using Kernel = void (*)(const Params);
    // [variant][0: bf16 out, 1: f32 out, 2: bf16 out into the gather buffers]: 0: batch <= 2, k 4096; 1: batch <= 2, k 2048;
    // 2: batch <= 4, k 4096; 3: batch <= 4, k 2048
    static const Kernel kernels[4][3] = {
        {int4_gemv_halfsm_kernel<1, 4, 8, false, false>, int4_gemv_halfsm_kernel<1, 4, 8, true, false>, int4_gemv_halfsm_kernel<1, 4, 8, false, true>},
        {int4_gemv_halfsm_kernel<1, 2, 8, false, false>, int4_gemv_halfsm_kernel<1, 2, 8, true, false>, int4_gemv_halfsm_kernel<1, 2, 8, false, true>},
        {int4_gemv_halfsm_kernel<2, 4, 8, false, false>, int4_gemv_halfsm_kernel<2, 4, 8, true, false>, int4_gemv_halfsm_kernel<2, 4, 8, false, true>},
        {int4_gemv_halfsm_kernel<2, 2, 8, false, false>, int4_gemv_halfsm_kernel<2, 2, 8, true, false>, int4_gemv_halfsm_kernel<2, 2, 8, false, true>}};
    // the residual block (norm in front, residual add behind): batch <= 2, bf16 outputs; [k 4096 | 2048]
    static const Kernel fused[2] = {int4_gemv_halfsm_kernel<1, 4, 8, false, false, false, true>,
                                    int4_gemv_halfsm_kernel<1, 2, 8, false, false, false, true>};
    const bool block = norm_w || resid || gate;
    if (block && (m > 2 || out_f32 || gather || (resid && gate))) return cudaErrorInvalidValue;
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        for (int i = 0; i < 14; ++i) {
            const void* f = i < 12 ? (const void*)kernels[i / 3][i % 3] : (const void*)fused[i - 12];
            cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (e != cudaSuccess) return e;
        }
        configured.fetch_or(bit, std::memory_order_release);
    }
    Params p{};
    p.norm_w = static_cast<const uint16_t*>(norm_w);
    p.norm_eps = norm_eps;
    p.resid = static_cast<const uint16_t*>(resid);
    p.gate = static_cast<const uint16_t*>(gate);
    p.x = static_cast<const uint16_t*>(x_bf16);
    p.w = static_cast<const uint8_t*>(w_packed);
    p.scales = static_cast<const uint16_t*>(scale_bf16);
    p.y = y;
    p.m = m;
    p.n = n;
    p.pace_ns = constant_weights ? PACE_NS : 0u;
    p.status = status;  // only the gathering form has a wait that can run out
    p.half = half & 1u;
    p.pipelined = pipelined ? 1u : 0u;
    if (gather) p.ag = *gather;
    // One CTA per SM, whole 16-row tiles each, the remainder spread one tile per CTA (14336 rows on 148 SMs: eight
    // CTAs with 7 tiles, the others with 6). Measured against 128 CTAs x 7 tiles and against two CTAs per SM (which
    // leave no room for the next launch): this split is the fastest.
    const uint32_t tiles = (n + TILE_ROWS - 1) / TILE_ROWS;
    const uint32_t grid = tiles < uint32_t(sm_count) ? tiles : uint32_t(sm_count);
    p.tiles_per_cta = tiles / grid;
    p.tiles_rem = tiles % grid;
    const int variant = (m <= 2 ? 0 : 2) + (k == 4096 ? 0 : 1);
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
    return cudaLaunchKernelEx(&cfg, block ? fused[k == 4096 ? 0 : 1] : kernels[variant][gather ? 2 : out_f32 ? 1 : 0], p);
}

// Rows longer than 4096: the k range is cut into blocks of 4096 (and one of 2048), each block is one launch of the k-block
// form of the kernel above over the strided sub-matrix, and every launch adds the f32 sums of the blocks before it in its
// reduction (the last one rounds to the output type). The launches form one programmatic chain like any other sequence of
// GEMVs. bf16 outputs accumulate in a stream-ordered scratch allocation, f32 outputs in the output itself.
bool int4_gemv_kblocks_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    return m >= 1 && m <= 4 && n >= 1 && group == 128 && k > 4096 && k % 2048 == 0;
}

namespace {
// The persistent workspace of the one-launch k split (per-tile arrival words, then the partial rows), one per (device,
// stream); made on first use outside stream capture, nullptr while the stream captures and none exists yet.
void* kblocks_workspace(int dev, cudaStream_t stream, size_t need) {
    struct Work {
        void* ptr;
        size_t bytes;
    };
    static std::mutex ws_mu;
    static std::map<std::pair<int, cudaStream_t>, Work> ws;
    std::lock_guard<std::mutex> lock(ws_mu);
    auto it = ws.find({dev, stream});
    if (it != ws.end() && it->second.bytes >= need) return it->second.ptr;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cudaGetLastError();
    if (cap != cudaStreamCaptureStatusNone) return nullptr;
    // a larger workspace replaces a smaller one; the old one may still be in use by launches in flight on this
    // stream and is kept (a handful of shapes per process)
    const size_t bytes = need < (size_t(8) << 20) ? (size_t(8) << 20) : need;
    void* fresh = nullptr;
    if (cudaMalloc(&fresh, bytes) == cudaSuccess && cudaMemsetAsync(fresh, 0, bytes, stream) == cudaSuccess) {
        ws[{dev, stream}] = Work{fresh, bytes};
        return fresh;
    }
    cudaGetLastError();
    if (fresh) cudaFree(fresh);
    return nullptr;
}
// The arrival words occupy a region of FIXED size at the start of the workspace and the partial rows follow it, whatever
// the shape: the words must be zero between launches, so no shape's partial sums may ever land where another shape (more
// rows, more tiles) keeps its words. 65536 words serve up to a million output rows; beyond that the launch-per-block
// form runs.
constexpr size_t KBLOCKS_COUNT_WORDS = size_t(1) << 16;
size_t kblocks_workspace_bytes(uint32_t m, uint32_t n, uint32_t k) {
    const uint32_t blk = k % 4096 == 0 ? 4096u : 2048u;
    return (KBLOCKS_COUNT_WORDS + size_t(k / blk) * m * n) * 4;
}
}  // namespace

cudaError_t launch_int4_gemv_kblocks(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                     uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                                     bool constant_weights, const void* resid, const void* gate, bool* stores_fused) {
    if (stores_fused) *stores_fused = false;
    if ((resid || gate) && (out_f32 || (resid && gate))) return cudaErrorInvalidValue;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    using Kernel = void (*)(const Params);
    // [batch <= 2 | <= 4][k block 4096 | 2048][bf16 | f32 out]
    static const Kernel kernels[2][2][2] = {
        {{int4_gemv_halfsm_kernel<1, 4, 8, false, false, true>, int4_gemv_halfsm_kernel<1, 4, 8, true, false, true>},
         {int4_gemv_halfsm_kernel<1, 2, 8, false, false, true>, int4_gemv_halfsm_kernel<1, 2, 8, true, false, true>}},
        {{int4_gemv_halfsm_kernel<2, 4, 8, false, false, true>, int4_gemv_halfsm_kernel<2, 4, 8, true, false, true>},
         {int4_gemv_halfsm_kernel<2, 2, 8, false, false, true>, int4_gemv_halfsm_kernel<2, 2, 8, true, false, true>}}};
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        for (int i = 0; i < 8; ++i) {
            const void* f = (const void*)kernels[i >> 2][(i >> 1) & 1][i & 1];
            e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(f, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (e != cudaSuccess) return e;
        }
        configured.fetch_or(bit, std::memory_order_release);
    }
    const uint32_t tiles = (n + TILE_ROWS - 1) / TILE_ROWS;
    // ---- one launch over all k blocks: needs a persistent workspace (partial rows and per-tile arrival words), one per
    // (device, stream); allocated on first use outside stream capture. A CTA takes the tiles of ONE k block, so it converts
    // one block of activations; the per-launch cost is paid once instead of once per block.
    {
        const uint32_t blk = k % 4096 == 0 ? 4096u : 2048u, kblocks = k / blk;
        const size_t count_words = KBLOCKS_COUNT_WORDS;  // arrival words first (fixed region), then the partial rows
        void* work = tiles <= KBLOCKS_COUNT_WORDS ? kblocks_workspace(dev, stream, kblocks_workspace_bytes(m, n, k)) : nullptr;
        if (work) {
            uint32_t* counts = static_cast<uint32_t*>(work);  // zero between launches: the last arriver of a tile resets its word
            float* part = reinterpret_cast<float*>(counts + count_words);
            {
                Params p{};
                p.x = static_cast<const uint16_t*>(x_bf16);
                p.w = static_cast<const uint8_t*>(w_packed);
                p.scales = static_cast<const uint16_t*>(scale_bf16);
                p.y = y;
                p.m = m;
                p.n = n;
                p.pace_ns = constant_weights ? PACE_NS : 0u;
                p.row_bytes = k / 2;
                p.scale_stride = k / 128;
                p.x_stride = k;
                p.kblocks = kblocks;
                p.part = part;
                p.tile_count = counts;
                p.resid = static_cast<const uint16_t*>(resid);  // applied where the last arriver rounds the sums
                p.gate = static_cast<const uint16_t*>(gate);
                if (stores_fused) *stores_fused = true;
                const uint64_t units = uint64_t(tiles) * kblocks;
                uint32_t grid = units < uint64_t(sm_count) ? uint32_t(units) : uint32_t(sm_count);
                if (grid < kblocks) grid = kblocks;
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
                return cudaLaunchKernelEx(&cfg, kernels[m <= 2 ? 0 : 1][blk == 4096 ? 0 : 1][out_f32 ? 1 : 0], p);
            }
        }
    }
    // ---- no workspace (first use under stream capture): one launch per k block
    float* sums = static_cast<float*>(y);  // f32 outputs accumulate in place
    if (!out_f32) {
        e = cudaMallocAsync(reinterpret_cast<void**>(&sums), size_t(m) * n * sizeof(float), stream);
        if (e != cudaSuccess) return e;
    }
    const uint32_t grid = tiles < uint32_t(sm_count) ? tiles : uint32_t(sm_count);
    for (uint32_t kb = 0; kb < k && e == cudaSuccess;) {
        const uint32_t blk = k - kb >= 4096 ? 4096u : 2048u;
        const bool last = kb + blk == k;
        Params p{};
        p.x = static_cast<const uint16_t*>(x_bf16) + kb;
        p.w = static_cast<const uint8_t*>(w_packed) + kb / 2;
        p.scales = static_cast<const uint16_t*>(scale_bf16) + kb / 128;
        p.y = last ? y : static_cast<void*>(sums);
        p.m = m;
        p.n = n;
        p.pace_ns = constant_weights ? PACE_NS : 0u;
        p.tiles_per_cta = tiles / grid;
        p.tiles_rem = tiles % grid;
        p.row_bytes = k / 2;
        p.scale_stride = k / 128;
        p.x_stride = k;
        p.acc_in = kb == 0 ? nullptr : sums;
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
        e = cudaLaunchKernelEx(&cfg, kernels[m <= 2 ? 0 : 1][blk == 4096 ? 0 : 1][(last ? out_f32 != 0 : true) ? 1 : 0], p);
        kb += blk;
    }
    if (!out_f32) {
        const cudaError_t fe = cudaFreeAsync(sums, stream);
        if (e == cudaSuccess) e = fe;
    }
    return e;
}

}  // namespace vybk
