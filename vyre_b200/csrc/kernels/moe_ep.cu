// Expert-parallel MoE FFN layer with device-side dispatch and combine over peer memory (NVLink), one process per GPU.
//
// Rank r owns experts [r * E/R, (r + 1) * E/R) and a share of the tokens. Per layer, all on the device and without a
// single host read-back:
//   route    router linear + gate for the local tokens (moe_ffn.cu)
//   count    per-expert histogram of the local routing; the row is stored into EVERY rank's count matrix [R][E]
//   plan     once all R rows have arrived: where this rank's rows start inside every expert's segment on the owner
//            (segments are padded to 256 rows; rows of lower ranks come first, token order inside a rank), and the
//            tile -> expert table of the local grouped GEMM
//   dispatch every (token, slot) row is stored straight into the owner's expert-sorted activation buffer, together
//            with its return address (source rank, pair index)
//   experts  once all R ranks have dispatched: grouped tensor-core GEMMs with the SwiGLU epilogue (CTA-pair kernel)
//   return   every result row is stored straight into the source rank's per-pair buffer
//   combine  once all R ranks have returned: weighted sum per token (moe_ffn.cu)
// Arrival is signalled by 32-bit counters that only grow (R arrivals per phase and layer); stores are fenced at system
// scope before the counter is bumped. Every wait is clock-bounded (~2 s) and raises status bit 256 instead of hanging.
// Buffers are reused by the next layer without extra handshakes: a rank starts layer s+1 only after every peer has
// returned its rows of layer s, which each peer does after it has finished reading everything this rank may
// overwrite. No multicast, no kernel of one GPU waits on another kernel of the same GPU.
//
// Reference semantics: vyre-libs/src/nn/moe/gating.rs:19-147, expert_mlp.rs:18-150, moe_layer.rs:33-121 (single-token
// ops; the sharding follows from experts being independent programs with disjoint weights).
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace vybk {
namespace {

constexpr uint32_t ROW_TILE = 256;
constexpr uint32_t MAX_EXPERTS = 64;
constexpr uint32_t MAX_TOPK = 8;
constexpr uint32_t PAD = 0xFFFFFFFFu;
constexpr long long WAIT_CLOCKS = 4000000000ll;
constexpr uint32_t FLAG_COUNT = 0, FLAG_DISPATCH = 16, FLAG_RETURN = 32;  // word offsets inside the flag block

// local (non-symmetric) control words
struct Local {
    uint32_t epoch;            // layers completed
    uint32_t ticket_dispatch;  // CTA tickets of the running dispatch / return kernels
    uint32_t ticket_return;
    uint32_t pad;
};

__device__ __forceinline__ uint8_t* sym(const MoeEp& c, uint32_t rank, unsigned long long off) {
    return reinterpret_cast<uint8_t*>(c.peer_base[rank] + off);
}
__device__ __forceinline__ uint32_t* flag_of(const MoeEp& c, uint32_t rank, uint32_t which) {
    return reinterpret_cast<uint32_t*>(sym(c, rank, c.off_flags)) + which;
}
// a wait that has run out once is not repeated: later calls return at once, so a broken run ends quickly with its
// status word set instead of spending the clock limit in every phase of every layer
__device__ bool wait_flag(const MoeEp& c, uint32_t which, uint32_t want, const uint32_t* status) {
    if (status && (*reinterpret_cast<const volatile uint32_t*>(status) & 256u)) return false;
    const volatile uint32_t* f = flag_of(c, c.rank, which);
    const long long limit = c.wait_clocks ? (long long)c.wait_clocks : WAIT_CLOCKS;
    const long long t0 = clock64();
    while (int32_t(*f - want) < 0) {
        if (clock64() - t0 > limit) return false;
        __nanosleep(64);
    }
    return true;
}
__device__ void signal_all(const MoeEp& c, uint32_t which) {
    for (uint32_t r = 0; r < c.world; ++r) atomicAdd_system(flag_of(c, r, which), 1u);
}

// ---- count: histogram of the local routing, published to every rank ---------------------------------------------------
__global__ void __launch_bounds__(1024)
ep_count_kernel(const MoeEp c, const uint32_t* __restrict__ idx, uint32_t pairs, uint32_t experts, uint32_t max_rows) {
    __shared__ uint32_t s_count[MAX_EXPERTS];
    if (threadIdx.x < MAX_EXPERTS) s_count[threadIdx.x] = 0;
    // return addresses of the local expert rows start as "padding"; sources fill them in after they have seen this
    // rank's counts, i.e. after the fence below
    uint2* src_info = reinterpret_cast<uint2*>(sym(c, c.rank, c.off_src));
    for (uint32_t i = threadIdx.x; i < max_rows; i += blockDim.x) src_info[i] = make_uint2(PAD, PAD);
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&s_count[idx[i]], 1u);
    __syncthreads();
    if (threadIdx.x < experts)
        for (uint32_t r = 0; r < c.world; ++r)
            reinterpret_cast<uint32_t*>(sym(c, r, c.off_counts))[c.rank * experts + threadIdx.x] = s_count[threadIdx.x];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) signal_all(c, FLAG_COUNT);
}

// ---- plan: destinations of the local rows and the local tile table -------------------------------------------------------
// plan words (local): [0] number of 256-row tiles, [1 .. 1 + E_local] segment starts, then tile_expert[max_tiles]
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const MoeEp c, const Local* __restrict__ local, const uint32_t* __restrict__ idx, uint32_t* __restrict__ plan,
               uint32_t* __restrict__ dst_row, uint32_t tokens, uint32_t topk, uint32_t experts, uint32_t* status) {
    __shared__ uint32_t s_counts[8][MAX_EXPERTS];
    __shared__ uint32_t s_base[MAX_EXPERTS], s_cursor[MAX_EXPERTS];
    __shared__ uint32_t s_warp_cnt[MAX_EXPERTS][32];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t el = experts / c.world;
    if (tid == 0 && !wait_flag(c, FLAG_COUNT, (local->epoch + 1) * c.world, status) && status) atomicOr(status, 256u);
    __syncthreads();
    const volatile uint32_t* counts = reinterpret_cast<const volatile uint32_t*>(sym(c, c.rank, c.off_counts));
    for (uint32_t i = tid; i < c.world * experts; i += blockDim.x) s_counts[i / experts][i % experts] = counts[i];
    if (tid < MAX_EXPERTS) s_cursor[tid] = 0;
    __syncthreads();
    if (tid == 0) {
        // every owner lays its experts out in order, each segment padded to whole tiles; inside a segment the rows
        // of rank 0 come first, then rank 1, ...
        uint32_t* tile_expert = plan + 2 + el;
        for (uint32_t d = 0; d < c.world; ++d) {
            uint32_t start = 0, tile = 0;
            for (uint32_t e = 0; e < el; ++e) {
                const uint32_t g = d * el + e;
                uint32_t total = 0, before = 0;
                for (uint32_t r = 0; r < c.world; ++r) {
                    if (r < c.rank) before += s_counts[r][g];
                    total += s_counts[r][g];
                }
                s_base[g] = start + before;
                const uint32_t padded = (total + ROW_TILE - 1) / ROW_TILE * ROW_TILE;
                if (d == c.rank) {
                    plan[1 + e] = start;
                    for (uint32_t t = 0; t < padded; t += ROW_TILE) tile_expert[tile++] = e;
                }
                start += padded;
            }
            if (d == c.rank) {
                plan[1 + el] = start;
                plan[0] = tile;
            }
        }
    }
    __syncthreads();
    // positions inside an expert keep token order (a token selects an expert at most once)
    for (uint32_t base = 0; base < tokens; base += blockDim.x) {
        const uint32_t t = base + tid;
        uint32_t my_e[MAX_TOPK], rank_in_warp[MAX_TOPK];
        for (uint32_t j = 0; j < MAX_TOPK; ++j) {
            my_e[j] = (j < topk && t < tokens) ? idx[size_t(t) * topk + j] : PAD;
            rank_in_warp[j] = 0;
        }
        for (uint32_t e = 0; e < experts; ++e) {
            bool sel = false;
            for (uint32_t j = 0; j < MAX_TOPK; ++j) sel |= (my_e[j] == e);
            const uint32_t b = __ballot_sync(0xffffffffu, sel);
            if (lane == 0) s_warp_cnt[e][warp] = __popc(b);
            const uint32_t rk = __popc(b & ((1u << lane) - 1u));
            for (uint32_t j = 0; j < MAX_TOPK; ++j)
                if (my_e[j] == e) rank_in_warp[j] = rk;
        }
        __syncthreads();
        for (uint32_t j = 0; j < MAX_TOPK; ++j) {
            const uint32_t e = my_e[j];
            if (e < experts) {
                uint32_t before = 0;
                for (uint32_t w = 0; w < warp; ++w) before += s_warp_cnt[e][w];
                dst_row[size_t(t) * topk + j] = s_base[e] + s_cursor[e] + before + rank_in_warp[j];
            }
        }
        __syncthreads();
        if (tid < experts) {
            uint32_t total = 0;
            for (uint32_t w = 0; w < 32; ++w) total += s_warp_cnt[tid][w];
            s_cursor[tid] += total;
        }
        __syncthreads();
    }
}

// last CTA of a multi-CTA kernel: all stores of all CTAs are fenced, then every rank's counter is bumped
__device__ void finish_phase(const MoeEp& c, uint32_t* ticket, uint32_t which) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t t = atomicAdd(ticket, 1u);
        if (t == gridDim.x - 1) {
            *reinterpret_cast<volatile uint32_t*>(ticket) = 0;
            __threadfence_system();
            signal_all(c, which);
        }
    }
}

// ---- dispatch: one warp per (token, slot) row, stored into the owner's expert-sorted buffer ---------------------------
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const MoeEp c, Local* local, const uint16_t* __restrict__ x, const uint32_t* __restrict__ idx,
                   const uint32_t* __restrict__ dst_row, uint32_t pairs, uint32_t topk, uint32_t experts, uint32_t hidden) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t el = experts / c.world;
    for (uint32_t p = blockIdx.x * 8 + warp; p < pairs; p += gridDim.x * 8) {
        const uint32_t owner = idx[p] / el, row = dst_row[p];
        const uint4* src = reinterpret_cast<const uint4*>(x + size_t(p / topk) * hidden);
        uint4* dst = reinterpret_cast<uint4*>(sym(c, owner, c.off_xg)) + size_t(row) * (hidden / 8);
        for (uint32_t i = lane; i < hidden / 8; i += 32) dst[i] = src[i];
        if (lane == 0) reinterpret_cast<uint2*>(sym(c, owner, c.off_src))[row] = make_uint2(c.rank, p);
    }
    finish_phase(c, &local->ticket_dispatch, FLAG_DISPATCH);
}

// ---- return: every valid local row goes back to the pair slot of its source rank --------------------------------------
__global__ void __launch_bounds__(256)
ep_return_kernel(const MoeEp c, Local* local, const uint16_t* __restrict__ y, const uint32_t* __restrict__ plan, uint32_t el,
                 uint32_t hidden) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rows = plan[1 + el];
    const uint2* src_info = reinterpret_cast<const uint2*>(sym(c, c.rank, c.off_src));
    for (uint32_t p = blockIdx.x * 8 + warp; p < rows; p += gridDim.x * 8) {
        const uint2 info = src_info[p];
        if (info.x == PAD) continue;
        const uint4* src = reinterpret_cast<const uint4*>(y + size_t(p) * hidden);
        uint4* dst = reinterpret_cast<uint4*>(sym(c, info.x, c.off_yhome)) + size_t(info.y) * (hidden / 8);
        for (uint32_t i = lane; i < hidden / 8; i += 32) dst[i] = src[i];
    }
    finish_phase(c, &local->ticket_return, FLAG_RETURN);
}

// ---- phase waits ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32)
ep_wait_kernel(const MoeEp c, Local* local, uint32_t which, uint32_t advance_epoch, uint32_t* status) {
    if (threadIdx.x != 0) return;
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(&local->epoch);
    if (!wait_flag(c, which, (e + 1) * c.world, status) && status) atomicOr(status, 256u);
    __threadfence_system();
    if (advance_epoch) *reinterpret_cast<volatile uint32_t*>(&local->epoch) = e + 1;
}

__global__ void identity_pos_kernel(uint32_t* pos, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) pos[i] = i;
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

uint32_t moe_ep_max_rows(uint32_t tokens_total, uint32_t experts, uint32_t topk, uint32_t world) {
    const uint64_t pairs = uint64_t(tokens_total) * topk;  // worst case: every pair of the whole job lands on one rank
    return uint32_t((pairs + ROW_TILE - 1) / ROW_TILE * ROW_TILE + uint64_t(experts / world) * ROW_TILE);
}

// symmetric region: counts, flags, return addresses, expert-sorted activations, per-pair results
void moe_ep_symmetric_layout(uint32_t tokens_local_max, uint32_t tokens_total, uint32_t hidden, uint32_t experts,
                             uint32_t topk, uint32_t world, MoeEp* c, size_t* total_bytes) {
    const uint32_t max_rows = moe_ep_max_rows(tokens_total, experts, topk, world);
    size_t off = 0;
    c->off_counts = off;
    off = align256(off + size_t(world) * experts * 4);
    c->off_flags = off;
    off = align256(off + 256);
    c->off_src = off;
    off = align256(off + size_t(max_rows) * 8);
    c->off_xg = off;
    off = align256(off + size_t(max_rows) * hidden * 2);
    c->off_yhome = off;
    off = align256(off + size_t(tokens_local_max) * topk * hidden * 2);
    *total_bytes = off;
}

size_t moe_ep_local_bytes(uint32_t tokens_local_max, uint32_t tokens_total, uint32_t hidden, uint32_t inter, uint32_t experts,
                          uint32_t topk, uint32_t world) {
    const uint32_t max_rows = moe_ep_max_rows(tokens_total, experts, topk, world);
    const size_t pairs = size_t(tokens_local_max) * topk;
    return 256 + align256(size_t(2 + experts / world + max_rows / ROW_TILE) * 4) + 2 * align256(pairs * 4) +
           align256(size_t(max_rows) * inter * 2) + align256(size_t(max_rows) * hidden * 2);
}

cudaError_t launch_moe_ep_ffn(const MoeEp& c, const void* x_bf16, const void* w_router_bf16, const void* w13, const void* s13,
                              const void* w2, const void* s2, void* out_bf16, uint32_t* routing_idx, float* routing_w,
                              void* local_scratch, uint32_t tokens, uint32_t tokens_total, uint32_t hidden, uint32_t inter,
                              uint32_t experts, uint32_t topk, uint32_t group, int sm_count, cudaStream_t stream,
                              uint32_t* status) {
    if (c.world < 1 || c.world > 8 || c.rank >= c.world || experts % c.world || experts > MAX_EXPERTS || topk > MAX_TOPK ||
        topk > experts || tokens == 0 || hidden % 256 || !moe_ffn_int4_supported(tokens, hidden, inter, experts / c.world, 1, group))
        return cudaErrorNotSupported;
    const uint32_t el = experts / c.world, pairs = tokens * topk;
    const uint32_t max_rows = moe_ep_max_rows(tokens_total, experts, topk, c.world);
    uint8_t* base = static_cast<uint8_t*>(local_scratch);
    Local* local = reinterpret_cast<Local*>(base);
    size_t off = 256;
    uint32_t* plan = reinterpret_cast<uint32_t*>(base + off);
    off += align256(size_t(2 + el + max_rows / ROW_TILE) * 4);
    uint32_t* dst_row = reinterpret_cast<uint32_t*>(base + off);
    off += align256(size_t(pairs) * 4);
    uint32_t* pos = reinterpret_cast<uint32_t*>(base + off);
    off += align256(size_t(pairs) * 4);
    uint16_t* h = reinterpret_cast<uint16_t*>(base + off);
    off += align256(size_t(max_rows) * inter * 2);
    uint16_t* y = reinterpret_cast<uint16_t*>(base + off);
    const uint16_t* xg = reinterpret_cast<const uint16_t*>(c.peer_base[c.rank] + c.off_xg);
    const uint16_t* y_home = reinterpret_cast<const uint16_t*>(c.peer_base[c.rank] + c.off_yhome);

    cudaError_t e = launch_moe_route(x_bf16, w_router_bf16, routing_idx, routing_w, tokens, hidden, experts, topk, stream);
    if (e != cudaSuccess) return e;
    ep_count_kernel<<<1, 1024, 0, stream>>>(c, routing_idx, pairs, experts, max_rows);
    ep_plan_kernel<<<1, 1024, 0, stream>>>(c, local, routing_idx, plan, dst_row, tokens, topk, experts, status);
    ep_dispatch_kernel<<<sm_count * 2, 256, 0, stream>>>(c, local, static_cast<const uint16_t*>(x_bf16), routing_idx, dst_row,
                                                         pairs, topk, experts, hidden);
    ep_wait_kernel<<<1, 32, 0, stream>>>(c, local, FLAG_DISPATCH, 0, status);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    e = launch_moe_experts_int4(xg, w13, s13, w2, s2, y, h, plan + 2 + el, plan, max_rows, hidden, inter, el, group, sm_count,
                                stream, status);
    if (e != cudaSuccess) return e;
    ep_return_kernel<<<sm_count * 2, 256, 0, stream>>>(c, local, y, plan, el, hidden);
    ep_wait_kernel<<<1, 32, 0, stream>>>(c, local, FLAG_RETURN, 1, status);
    identity_pos_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(pos, pairs);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    return launch_moe_combine(y_home, pos, routing_w, out_bf16, tokens, hidden, topk, sm_count, stream);
}

}  // namespace vybk
