// Multi-token int4 MoE FFN layer: router + softmax top-k gate, expert-sorted token permutation, grouped expert
// GEMMs (SwiGLU fused into the first), weighted combine.
//
//   logits[t, e] = bf16( x[t, :] . w_router[e, :] )                      f32 accumulate
//   (idx, w)[t]  = moe_gate(f32(logits[t, :]), k)                        softmax over ALL experts, strict-'>' top-k
//   h[p, :]      = swiglu( x[t(p)] . W1[e(p)]^T, x[t(p)] . W3[e(p)]^T )  bf16, tcgen05 grouped GEMM
//   y[p, :]      = bf16( h[p, :] . W2[e(p)]^T )                          tcgen05 grouped GEMM
//   out[t, :]    = bf16( sum_j w[t, j] * f32(y[pos(t, j), :]) )          sequential over the k slots
//
// Rows are sorted by expert; each expert's segment starts on a 256-row boundary so that no 256-row GEMM tile
// (one CTA pair) straddles two experts; a small table gives the expert of each tile and a device word the number of
// tiles, so the GEMM launches are shaped on the device and the host never reads the routing back.
//
// Per-token semantics follow vyre-libs/src/nn/moe/gating.rs:19-147 (gate), vyre-libs/src/nn/moe/expert_mlp.rs:18-150
// with vyre-libs/src/nn/activation/swiglu.rs:26 (expert), vyre-libs/src/nn/moe/moe_layer.rs:33-121 (combine); the
// reference ops are single-token, this is their batched composition.
#include <cuda_bf16.h>

#include <algorithm>
#include <float.h>

#include "kernels.h"

namespace vybk {
namespace {

constexpr uint32_t ROW_TILE = 256;       // rows per CTA-pair tile of the grouped GEMM
constexpr uint32_t MAX_EXPERTS = 64;
constexpr uint32_t MAX_TOPK = 8;
constexpr uint32_t PAD_TOKEN = 0xFFFFFFFFu;

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b) { return __uint_as_float(b << 16); }

// ---- router + gate: one warp per token; a CTA keeps the router weights in shared memory and walks many tokens -------
template <bool WR_IN_SMEM>
__global__ void __launch_bounds__(256, 2)
moe_router_gate_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w_router, uint32_t* __restrict__ idx,
                       float* __restrict__ wts, uint32_t tokens, uint32_t hidden, uint32_t experts, uint32_t topk) {
    extern __shared__ __align__(16) uint8_t s_dyn[];
    __shared__ float s_logits[8][MAX_EXPERTS];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint16_t* wr = w_router;
    if constexpr (WR_IN_SMEM) {
        uint4* dst = reinterpret_cast<uint4*>(s_dyn);
        const uint4* src = reinterpret_cast<const uint4*>(w_router);
        for (uint32_t i = threadIdx.x; i < experts * hidden / 8; i += blockDim.x) dst[i] = src[i];
        __syncthreads();
        wr = reinterpret_cast<const uint16_t*>(s_dyn);
    }
    for (uint32_t t = blockIdx.x * 8 + warp; t < tokens; t += gridDim.x * 8) {
    const uint16_t* xr = x + size_t(t) * hidden;
    // The token's row is fetched whole before any arithmetic (up to 16 independent 16-byte loads per lane, 8 K elements
    // per warp): with one load per 256-element step, as before, a token cost sixteen dependent trips to L2 / HBM. The
    // arithmetic order is unchanged (a lane sums its own elements in k order, lanes fold by shuffles).
    constexpr uint32_t XCHUNKS = 16;
    uint4 xrow[XCHUNKS];
    const uint32_t nchunks = (hidden + 255) / 256;
    if (nchunks <= XCHUNKS) {
#pragma unroll
        for (uint32_t c = 0; c < XCHUNKS; ++c) {
            const uint32_t k = c * 256 + lane * 8;
            xrow[c] = k < hidden ? __ldg(reinterpret_cast<const uint4*>(xr + k)) : make_uint4(0, 0, 0, 0);
        }
    }
    for (uint32_t e0 = 0; e0 < experts; e0 += 8) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const uint32_t ne = min(8u, experts - e0);
#pragma unroll
        for (uint32_t c = 0; c < XCHUNKS; ++c) {
            const uint32_t k = c * 256 + lane * 8;  // hidden % 8 == 0
            if (nchunks <= XCHUNKS && k < hidden) {
                const uint4 xv = xrow[c];
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (uint32_t e = 0; e < 8; ++e) {
                    if (e < ne) {
                        const uint4 wv = *reinterpret_cast<const uint4*>(wr + size_t(e0 + e) * hidden + k);
                        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            acc[e] = fmaf(bf16_bits_to_float(xw[q] & 0xFFFFu), bf16_bits_to_float(ww[q] & 0xFFFFu), acc[e]);
                            acc[e] = fmaf(bf16_bits_to_float(xw[q] >> 16), bf16_bits_to_float(ww[q] >> 16), acc[e]);
                        }
                    }
                }
            }
        }
        if (nchunks > XCHUNKS) {  // rows longer than 4096 elements: the plain loop
            for (uint32_t k = lane * 8; k < hidden; k += 256) {
                const uint4 xv = *reinterpret_cast<const uint4*>(xr + k);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (uint32_t e = 0; e < 8; ++e) {
                    if (e < ne) {
                        const uint4 wv = *reinterpret_cast<const uint4*>(wr + size_t(e0 + e) * hidden + k);
                        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            acc[e] = fmaf(bf16_bits_to_float(xw[q] & 0xFFFFu), bf16_bits_to_float(ww[q] & 0xFFFFu), acc[e]);
                            acc[e] = fmaf(bf16_bits_to_float(xw[q] >> 16), bf16_bits_to_float(ww[q] >> 16), acc[e]);
                        }
                    }
                }
            }
        }
#pragma unroll
        for (uint32_t e = 0; e < 8; ++e) {
            float v = acc[e];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && e < ne) s_logits[warp][e0 + e] = __bfloat162float(__float2bfloat16_rn(v));  // logits are bf16
        }
    }
    __syncwarp();
    if (lane == 0) {
        // gate on the f32 view of the bf16 logits, in the reference's order
        float* sc = s_logits[warp];
        float mx = -FLT_MAX;
        for (uint32_t e = 0; e < experts; ++e) mx = fmaxf(mx, sc[e]);
        float sum = 0.0f;
        for (uint32_t e = 0; e < experts; ++e) sum = __fadd_rn(sum, expf(__fsub_rn(sc[e], mx)));
        uint32_t best_idx[MAX_TOPK];
        float best_val[MAX_TOPK];
        for (uint32_t j = 0; j < topk; ++j) {
            uint32_t best = 0;
            float bs = -FLT_MAX;
            for (uint32_t e = 0; e < experts; ++e)
                if (sc[e] > bs) {
                    bs = sc[e];
                    best = e;
                }
            best_idx[j] = best;
            best_val[j] = bs;
            sc[best] = -FLT_MAX;  // sentinel: the winner leaves the race
        }
        for (uint32_t j = 0; j < topk; ++j) {
            idx[size_t(t) * topk + j] = best_idx[j];
            wts[size_t(t) * topk + j] = __fdiv_rn(expf(__fsub_rn(best_val[j], mx)), sum);
        }
    }
    __syncwarp();
    }  // token loop
}

// the router weights stay in shared memory when they fit beside the other kernels' carve-out
constexpr size_t ROUTER_SMEM_LIMIT = 160 * 1024;
cudaError_t launch_router_gate(const uint16_t* x, const uint16_t* w_router, uint32_t* idx, float* wts, uint32_t tokens,
                               uint32_t hidden, uint32_t experts, uint32_t topk, int sm_count, cudaStream_t stream) {
    const size_t wr_bytes = size_t(experts) * hidden * 2;
    const uint32_t want_blocks = (tokens + 7) / 8;
    if (wr_bytes <= ROUTER_SMEM_LIMIT) {
        static bool configured[64] = {};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (!configured[dev & 63]) {
            e = cudaFuncSetAttribute(moe_router_gate_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(ROUTER_SMEM_LIMIT));
            if (e != cudaSuccess) return e;
            configured[dev & 63] = true;
        }
        const uint32_t per_sm = uint32_t(std::max<size_t>(1, std::min<size_t>(2, (200 * 1024) / std::max<size_t>(wr_bytes, 1))));
        const uint32_t grid = min(want_blocks, uint32_t(sm_count) * per_sm);
        moe_router_gate_kernel<true><<<grid, 256, wr_bytes, stream>>>(x, w_router, idx, wts, tokens, hidden, experts, topk);
    } else {
        moe_router_gate_kernel<false><<<want_blocks, 256, 0, stream>>>(x, w_router, idx, wts, tokens, hidden, experts, topk);
    }
    return cudaGetLastError();
}

// ---- plan: expert segments, tile table, deterministic row positions (single CTA) -------------------------------------
// plan words: [0] number of 256-row tiles, [1 .. 1+E] segment starts (rows), then tile_expert[max_tiles].
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const uint32_t* __restrict__ idx, uint32_t* __restrict__ plan, uint32_t* __restrict__ pos,
                uint32_t* __restrict__ row_token, uint32_t tokens, uint32_t experts, uint32_t topk, uint32_t max_rows) {
    __shared__ uint32_t s_count[MAX_EXPERTS], s_start[MAX_EXPERTS + 1], s_cursor[MAX_EXPERTS];
    __shared__ uint32_t s_warp_cnt[MAX_EXPERTS][32];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < MAX_EXPERTS) {
        s_count[tid] = 0;
        s_cursor[tid] = 0;
    }
    for (uint32_t i = tid; i < max_rows; i += blockDim.x) row_token[i] = PAD_TOKEN;
    __syncthreads();
    for (uint32_t i = tid; i < tokens * topk; i += blockDim.x) atomicAdd(&s_count[idx[i]], 1u);
    __syncthreads();
    if (tid == 0) {
        uint32_t start = 0, tile = 0;
        uint32_t* tile_expert = plan + 2 + experts;
        for (uint32_t e = 0; e < experts; ++e) {
            s_start[e] = start;
            plan[1 + e] = start;
            const uint32_t padded = (s_count[e] + ROW_TILE - 1) / ROW_TILE * ROW_TILE;
            for (uint32_t r = 0; r < padded; r += ROW_TILE) tile_expert[tile++] = e;
            start += padded;
        }
        s_start[experts] = start;
        plan[1 + experts] = start;
        plan[0] = tile;
    }
    __syncthreads();
    // positions: rows of an expert keep token order (a token selects an expert at most once)
    for (uint32_t base = 0; base < tokens; base += blockDim.x) {
        const uint32_t t = base + tid;
        uint32_t my_e[MAX_TOPK], rank_in_warp[MAX_TOPK];
        for (uint32_t j = 0; j < MAX_TOPK; ++j) {
            my_e[j] = (j < topk && t < tokens) ? idx[size_t(t) * topk + j] : 0xFFFFFFFFu;
            rank_in_warp[j] = 0;
        }
        for (uint32_t e = 0; e < experts; ++e) {  // warp-uniform loop: every lane votes for every expert
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
                const uint32_t p = s_start[e] + s_cursor[e] + before + rank_in_warp[j];
                pos[size_t(t) * topk + j] = p;
                row_token[p] = t;
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

// ---- gather: expert-sorted activation rows (padding rows are zero) ---------------------------------------------------
__global__ void __launch_bounds__(256)
moe_gather_kernel(const uint16_t* __restrict__ x, const uint32_t* __restrict__ row_token, const uint32_t* __restrict__ plan,
                  uint16_t* __restrict__ xg, uint32_t hidden, uint32_t experts) {
    const uint32_t rows = plan[1 + experts];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t p = blockIdx.x * 8 + warp; p < rows; p += gridDim.x * 8) {
        const uint32_t t = row_token[p];
        uint4* dst = reinterpret_cast<uint4*>(xg + size_t(p) * hidden);
        if (t == PAD_TOKEN) {
            for (uint32_t c = lane; c < hidden / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(x + size_t(t) * hidden);
            for (uint32_t c = lane; c < hidden / 8; c += 32) dst[c] = src[c];
        }
    }
}

// ---- combine: out[t] = bf16( sum_j w[t,j] * y[pos[t,j]] ), slots in selection order, separate multiply and add -------
__global__ void __launch_bounds__(256)
moe_combine_kernel(const uint16_t* __restrict__ y, const uint32_t* __restrict__ pos, const float* __restrict__ wts,
                   uint16_t* __restrict__ out, uint32_t tokens, uint32_t hidden, uint32_t topk) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t t = blockIdx.x * 8 + warp; t < tokens; t += gridDim.x * 8) {
        for (uint32_t c = lane; c < hidden / 8; c += 32) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (uint32_t j = 0; j < topk; ++j) {
                const float w = wts[size_t(t) * topk + j];
                const uint4 v = reinterpret_cast<const uint4*>(y + size_t(pos[size_t(t) * topk + j]) * hidden)[c];
                const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    acc[2 * q] = __fadd_rn(acc[2 * q], __fmul_rn(w, bf16_bits_to_float(vw[q] & 0xFFFFu)));
                    acc[2 * q + 1] = __fadd_rn(acc[2 * q + 1], __fmul_rn(w, bf16_bits_to_float(vw[q] >> 16)));
                }
            }
            uint32_t pk[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
                pk[q] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            reinterpret_cast<uint4*>(out + size_t(t) * hidden)[c] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
}

// ---- generic row gather: dst[i, :] = src[index[i], :], zeros where index[i] is the padding marker --------------------
__global__ void __launch_bounds__(256)
rows_gather_kernel(const uint16_t* __restrict__ src, const uint32_t* __restrict__ index, uint16_t* __restrict__ dst,
                   uint32_t rows, uint32_t row_elems) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t p = blockIdx.x * 8 + warp; p < rows; p += gridDim.x * 8) {
        const uint32_t t = index[p];
        uint4* d = reinterpret_cast<uint4*>(dst + size_t(p) * row_elems);
        if (t == PAD_TOKEN) {
            for (uint32_t c = lane; c < row_elems / 8; c += 32) d[c] = make_uint4(0, 0, 0, 0);
        } else {
            const uint4* sp = reinterpret_cast<const uint4*>(src + size_t(t) * row_elems);
            for (uint32_t c = lane; c < row_elems / 8; c += 32) d[c] = sp[c];
        }
    }
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

struct Layout {
    uint32_t max_rows, max_tiles;
    size_t plan, pos, row_token, xg, h, y, total;
};

Layout layout_for(uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t topk) {
    Layout L{};
    const uint64_t pairs = uint64_t(tokens) * topk;
    L.max_rows = uint32_t((pairs + ROW_TILE - 1) / ROW_TILE * ROW_TILE + uint64_t(experts) * ROW_TILE);
    L.max_tiles = L.max_rows / ROW_TILE;
    size_t off = 0;
    L.plan = off;
    off = align256(off + size_t(2 + experts + L.max_tiles) * 4);
    L.pos = off;
    off = align256(off + size_t(pairs) * 4);
    L.row_token = off;
    off = align256(off + size_t(L.max_rows) * 4);
    L.xg = off;
    off = align256(off + size_t(L.max_rows) * hidden * 2);
    L.h = off;
    off = align256(off + size_t(L.max_rows) * inter * 2);
    L.y = off;
    off = align256(off + size_t(L.max_rows) * hidden * 2);
    L.total = off;
    return L;
}

}  // namespace

bool moe_ffn_int4_supported(uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t topk,
                            uint32_t group) {
    return tokens >= 1 && experts >= 1 && experts <= MAX_EXPERTS && topk >= 1 && topk <= MAX_TOPK && topk <= experts &&
           hidden % 256 == 0 && inter % 256 == 0 && group >= 64 && group % 64 == 0 && hidden % group == 0 &&
           inter % group == 0;
}

size_t moe_ffn_int4_scratch_bytes(uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t topk) {
    return layout_for(tokens, hidden, inter, experts, topk).total;
}

cudaError_t launch_moe_ffn_int4(const void* x_bf16, const void* w_router_bf16, const void* w13, const void* s13,
                                const void* w2, const void* s2, void* out_bf16, uint32_t* routing_idx, float* routing_w,
                                void* scratch, uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts,
                                uint32_t topk, uint32_t group, int sm_count, cudaStream_t stream, uint32_t* status) {
    if (!moe_ffn_int4_supported(tokens, hidden, inter, experts, topk, group)) return cudaErrorNotSupported;
    const Layout L = layout_for(tokens, hidden, inter, experts, topk);
    uint8_t* base = static_cast<uint8_t*>(scratch);
    uint32_t* plan = reinterpret_cast<uint32_t*>(base + L.plan);
    uint32_t* pos = reinterpret_cast<uint32_t*>(base + L.pos);
    uint32_t* row_token = reinterpret_cast<uint32_t*>(base + L.row_token);
    uint16_t* xg = reinterpret_cast<uint16_t*>(base + L.xg);
    uint16_t* h = reinterpret_cast<uint16_t*>(base + L.h);
    uint16_t* y = reinterpret_cast<uint16_t*>(base + L.y);
    const uint32_t* tile_expert = plan + 2 + experts;

    cudaError_t e = launch_router_gate(static_cast<const uint16_t*>(x_bf16), static_cast<const uint16_t*>(w_router_bf16),
                                       routing_idx, routing_w, tokens, hidden, experts, topk, sm_count, stream);
    if (e != cudaSuccess) return e;
    moe_plan_kernel<<<1, 1024, 0, stream>>>(routing_idx, plan, pos, row_token, tokens, experts, topk, L.max_rows);
    moe_gather_kernel<<<sm_count * 4, 256, 0, stream>>>(static_cast<const uint16_t*>(x_bf16), row_token, plan, xg, hidden,
                                                        experts);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    // h = swiglu(xg . W1^T, xg . W3^T) per expert
    e = launch_int4_gemm_pair(xg, w13, s13, h, L.max_rows, inter, hidden, group, 0, 1, experts, tile_expert, plan, inter,
                              sm_count, stream, status);
    if (e != cudaSuccess) return e;
    // y = h . W2^T per expert
    e = launch_int4_gemm_pair(h, w2, s2, y, L.max_rows, hidden, inter, group, 0, 0, experts, tile_expert, plan, hidden,
                              sm_count, stream, status);
    if (e != cudaSuccess) return e;
    moe_combine_kernel<<<sm_count * 4, 256, 0, stream>>>(y, pos, routing_w, static_cast<uint16_t*>(out_bf16), tokens,
                                                         hidden, topk);
    return cudaGetLastError();
}

// ---- the stages on their own, for expert-parallel runs where an exchange sits between them ---------------------------
cudaError_t launch_moe_route(const void* x_bf16, const void* w_router_bf16, uint32_t* routing_idx, float* routing_w,
                             uint32_t tokens, uint32_t hidden, uint32_t experts, uint32_t topk, cudaStream_t stream) {
    if (tokens == 0 || experts == 0 || experts > MAX_EXPERTS || topk == 0 || topk > MAX_TOPK || topk > experts || hidden % 8)
        return cudaErrorNotSupported;
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    return launch_router_gate(static_cast<const uint16_t*>(x_bf16), static_cast<const uint16_t*>(w_router_bf16), routing_idx,
                              routing_w, tokens, hidden, experts, topk, sms, stream);
}

cudaError_t launch_rows_gather_bf16(const void* src, const uint32_t* index, void* dst, uint32_t rows, uint32_t row_elems,
                                    int sm_count, cudaStream_t stream) {
    if (row_elems % 8) return cudaErrorNotSupported;
    if (rows == 0) return cudaSuccess;
    rows_gather_kernel<<<sm_count * 4, 256, 0, stream>>>(static_cast<const uint16_t*>(src), index,
                                                         static_cast<uint16_t*>(dst), rows, row_elems);
    return cudaGetLastError();
}

// rows: expert-sorted, every expert's segment padded to 256 rows; plan[0] = number of 256-row tiles (device word),
// tile_expert[i] = local expert of tile i. h_scratch holds [max_rows, inter] bf16.
cudaError_t launch_moe_experts_int4(const void* x_sorted, const void* w13, const void* s13, const void* w2, const void* s2,
                                    void* y_rows, void* h_scratch, const uint32_t* tile_expert, const uint32_t* m_tiles_dev,
                                    uint32_t max_rows, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t group,
                                    int sm_count, cudaStream_t stream, uint32_t* status) {
    if (max_rows == 0 || max_rows % ROW_TILE || !moe_ffn_int4_supported(1, hidden, inter, experts, 1, group))
        return cudaErrorNotSupported;
    cudaError_t e = launch_int4_gemm_pair(x_sorted, w13, s13, h_scratch, max_rows, inter, hidden, group, 0, 1, experts,
                                          tile_expert, m_tiles_dev, inter, sm_count, stream, status);
    if (e != cudaSuccess) return e;
    return launch_int4_gemm_pair(h_scratch, w2, s2, y_rows, max_rows, hidden, inter, group, 0, 0, experts, tile_expert,
                                 m_tiles_dev, hidden, sm_count, stream, status);
}

cudaError_t launch_moe_combine(const void* y_rows, const uint32_t* pos, const float* routing_w, void* out_bf16,
                               uint32_t tokens, uint32_t hidden, uint32_t topk, int sm_count, cudaStream_t stream) {
    if (hidden % 8 || topk == 0 || topk > MAX_TOPK) return cudaErrorNotSupported;
    if (tokens == 0) return cudaSuccess;
    moe_combine_kernel<<<sm_count * 4, 256, 0, stream>>>(static_cast<const uint16_t*>(y_rows), pos, routing_w,
                                                         static_cast<uint16_t*>(out_bf16), tokens, hidden, topk);
    return cudaGetLastError();
}

}  // namespace vybk
