// Small operators of the vyre-libs NN / quant surface, each evaluated in the reference interpreter's own
// order so that f32 results are bit-identical to it (subnormals flush like the interpreter's
// canonicalisation because this file is compiled with -ftz=true; mul/add never contract because every step
// uses the explicit-rounding intrinsics). These are latency-sized ops (routers, activations, fixtures), not
// the bandwidth- or tensor-bound kernels, which live in their own files.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <float.h>

#include "kernels.h"

namespace vybk {
namespace {

__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }

__device__ __forceinline__ int32_t i4_lane(const uint32_t* packed, uint32_t lane) {
    const uint32_t nib = (packed[lane >> 3] >> ((lane & 7) * 4)) & 0xFu;
    return (nib & 8u) ? int32_t(nib) - 16 : int32_t(nib);
}

// dtype: 0 f32, 1 bf16, 2 f16 (conversion rules of vyre-reference/src/float16.rs)
__device__ __forceinline__ float load_typed(const void* p, size_t i, uint32_t dt) {
    if (dt == 1) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    if (dt == 2) return __half2float(static_cast<const __half*>(p)[i]);
    return static_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_typed(void* p, size_t i, uint32_t dt, float v) {
    if (dt == 1)
        static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else if (dt == 2)
        static_cast<__half*>(p)[i] = __float2half_rn(v);
    else
        static_cast<float*>(p)[i] = v;
}

// vyre-libs/src/nn/linear/inner/linear_4bit.rs:255-335: thread per output, sequential k, mul then add.
__global__ void linear_4bit_kernel(const float* x, const uint32_t* w, const float* b, float* out, uint32_t in_dim,
                                   uint32_t out_dim) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= out_dim) return;
    float acc = b[i];
    for (uint32_t k = 0; k < in_dim; ++k) {
        const uint32_t word = w[size_t(k >> 3) * out_dim + i];
        acc = fadd(acc, fmul(x[k], float((word >> ((k & 7) * 4)) & 0xFu)));
    }
    out[i] = acc;
}

// linear_4bit.rs:505-708: one warp per (batch, output); lane l runs the FMA chain over k = 32c + l, the
// warp sum folds lanes 0..31 in order from 0.0 (vyre-reference/src/execution/hashmap/subgroup.rs:87-117).
__global__ void affine_grouped_kernel(const float* x, const uint32_t* w, const float* scale, const uint32_t* zp,
                                      const float* b, float* out, uint32_t in_dim, uint32_t out_dim, uint32_t group,
                                      uint32_t total) {
    const uint32_t o = blockIdx.x * 8 + (threadIdx.x >> 5);
    const uint32_t lane = threadIdx.x & 31;
    if (o >= total) return;
    const uint32_t bi = o / out_dim, i = o % out_dim;
    const float* xb = x + size_t(bi) * in_dim;
    float acc = 0.0f;
    for (uint32_t k = lane; k < in_dim; k += 32) {
        const uint32_t word = w[size_t(k >> 3) * out_dim + i];
        const float nib = float((word >> ((k & 7) * 4)) & 0xFu);
        const size_t side = size_t(k / group) * out_dim + i;
        const float s = scale[side];
        const float neg_s = __fmaf_rn(-1.0f, s, -0.0f);
        const float zero_off = __fmaf_rn(float(zp[side]), neg_s, -0.0f);
        acc = __fmaf_rn(xb[k], __fmaf_rn(nib, s, zero_off), acc);
    }
    float sum = 0.0f;
    for (int l = 0; l < 32; ++l) sum = fadd(sum, __shfl_sync(0xffffffffu, acc, l));
    if (lane == 0) out[o] = fadd(b[i], sum);
}

__global__ void i4_unpack_kernel(const uint32_t* packed, int32_t* out, uint32_t lanes) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < lanes) out[t] = i4_lane(packed, t);
}
__global__ void i4_dot_i32_kernel(const uint32_t* lhs, const uint32_t* rhs, int32_t* out, uint32_t lanes) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    uint32_t acc = 0;
    for (uint32_t l = 0; l < lanes; ++l) acc += uint32_t(i4_lane(lhs, l)) * uint32_t(i4_lane(rhs, l));
    out[0] = int32_t(acc);
}
__global__ void i4_dot_f32_scaled_kernel(const uint32_t* lhs, const uint32_t* rhs, const float* ls, const float* rs,
                                         float* out, uint32_t lanes) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    float acc = 0.0f;
    for (uint32_t l = 0; l < lanes; ++l) acc = fadd(acc, fmul(float(i4_lane(lhs, l)), float(i4_lane(rhs, l))));
    out[0] = fmul(fmul(acc, ls[0]), rs[0]);
}
// vyre-primitives/src/math/quantized/program_helpers.rs:7-81
__global__ void i4_batched_matvec_kernel(const uint32_t* w, const float* x, const float* scales, float* out,
                                         uint32_t batch, uint32_t rows, uint32_t cols) {
    const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= batch * rows) return;
    const uint32_t row = item % rows, b = item / rows;
    const uint32_t wpr = (cols + 7) / 8;
    const uint32_t* wr = w + size_t(row) * wpr;
    const float* xb = x + size_t(b) * cols;
    float acc = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) acc = fadd(acc, fmul(float(i4_lane(wr, c)), xb[c]));
    out[item] = fmul(acc, scales[row]);
}
// programs.rs:309-456
__global__ void i4_batched_matmul_kernel(const uint32_t* w, const uint32_t* act, const float* rs, const float* bs,
                                         float* out, uint32_t batch, uint32_t rows, uint32_t cols) {
    const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= batch * rows) return;
    const uint32_t row = item % rows, b = item / rows;
    const uint32_t wpr = (cols + 7) / 8;
    const uint32_t* wr = w + size_t(row) * wpr;
    const uint32_t* ab = act + size_t(b) * wpr;
    float acc = 0.0f;
    for (uint32_t c = 0; c < cols; ++c) acc = fadd(acc, fmul(float(i4_lane(wr, c)), float(i4_lane(ab, c))));
    out[item] = fmul(fmul(acc, rs[row]), bs[b]);
}
// programs.rs:457-616: strict '<' update, init f32::MIN, out = [scores | f32(index)]
__global__ void i4_batched_matmul_top1_kernel(const uint32_t* w, const uint32_t* act, const float* rs,
                                              const float* bs, float* out, uint32_t batch, uint32_t rows,
                                              uint32_t cols) {
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    const uint32_t wpr = (cols + 7) / 8;
    const uint32_t* ab = act + size_t(b) * wpr;
    float best = -FLT_MAX;
    uint32_t best_idx = 0;
    for (uint32_t row = 0; row < rows; ++row) {
        const uint32_t* wr = w + size_t(row) * wpr;
        float acc = 0.0f;
        for (uint32_t c = 0; c < cols; ++c) acc = fadd(acc, fmul(float(i4_lane(wr, c)), float(i4_lane(ab, c))));
        const float score = fmul(fmul(acc, rs[row]), bs[b]);
        if (best < score) {
            best = score;
            best_idx = row;
        }
    }
    out[b] = best;
    out[batch + b] = float(best_idx);
}

// vyre-libs/src/nn/quant/int8.rs:15-78
__global__ void int8_unpack_kernel(const uint32_t* packed, const float* scales, float* out, uint32_t n, uint32_t cols) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = fmul(float(packed[i]), scales[i / cols]);
}
__global__ void int8_pack_kernel(const uint32_t* in, uint32_t* out, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i] & 0xFFu;
}

// vyre-libs/src/nn/linear/inner/builder.rs:287-344
__global__ void linear_rows_kernel(const void* x, const void* w, const void* bias, void* out, uint32_t rows,
                                   uint32_t in_dim, uint32_t out_dim, uint32_t dt, uint32_t out_in) {
    const uint32_t index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= rows * out_dim) return;
    const uint32_t row = index / out_dim, col = index % out_dim;
    float acc = bias ? load_typed(bias, col, dt) : 0.0f;
    for (uint32_t k = 0; k < in_dim; ++k) {
        const size_t wi = out_in ? size_t(col) * in_dim + k : size_t(k) * out_dim + col;
        acc = fadd(acc, fmul(load_typed(x, size_t(row) * in_dim + k, dt), load_typed(w, wi, dt)));
    }
    store_typed(out, index, dt, acc);
}

// vyre-libs/src/math/linalg/matmul.rs:17-60 (matmul), :138-271,330-380 (matmul_bias: out = acc + bias[col]); the same
// result serves nn::linear (m = 1; vyre-libs/src/nn/linear/inner/builder.rs:363-391) and the tiled forms
// (matmul_tiled/program.rs). u32 arithmetic wraps, so every summation order gives the same bits: 32x32 output tiles,
// operands staged in shared memory 32 k at a time.
__global__ void __launch_bounds__(256) matmul_u32_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b,
                                                         const uint32_t* __restrict__ bias, uint32_t* __restrict__ out,
                                                         uint32_t m, uint32_t k, uint32_t n) {
    __shared__ uint32_t as[32][33], bs[32][33];
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 8 row groups x 32 columns; 4 rows per thread
    const uint32_t row0 = blockIdx.y * 32, col0 = blockIdx.x * 32;
    uint32_t acc[4] = {0, 0, 0, 0};
    for (uint32_t k0 = 0; k0 < k; k0 += 32) {
        for (uint32_t r = ty; r < 32; r += 8) {
            as[r][tx] = (row0 + r < m && k0 + tx < k) ? a[size_t(row0 + r) * k + k0 + tx] : 0u;
            bs[r][tx] = (k0 + r < k && col0 + tx < n) ? b[size_t(k0 + r) * n + col0 + tx] : 0u;
        }
        __syncthreads();
#pragma unroll 8
        for (uint32_t kk = 0; kk < 32; ++kk) {
            const uint32_t bv = bs[kk][tx];
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[r] += as[ty + 8 * r][kk] * bv;
        }
        __syncthreads();
    }
    const uint32_t col = col0 + tx;
    if (col >= n) return;
    const uint32_t bv = bias ? bias[col] : 0u;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t row = row0 + ty + 8 * r;
        if (row < m) out[size_t(row) * n + col] = acc[r] + bv;
    }
}

// vyre-libs/src/nn/moe/gating.rs:71-147; one thread per token, experts staged in shared memory
__global__ void moe_gate_kernel(const float* scores, uint32_t* idx, float* weights, uint32_t tokens, uint32_t experts,
                                uint32_t k) {
    extern __shared__ float scratch_all[];
    const uint32_t tok = blockIdx.x * blockDim.x + threadIdx.x;
    if (tok >= tokens) return;
    float* scratch = scratch_all + size_t(threadIdx.x) * experts;
    const float* s = scores + size_t(tok) * experts;
    float mx = -FLT_MAX;
    for (uint32_t i = 0; i < experts; ++i) {
        scratch[i] = s[i];
        mx = fmaxf(mx, s[i]);
    }
    float sum = 0.0f;
    for (uint32_t i = 0; i < experts; ++i) sum = fadd(sum, expf(__fsub_rn(s[i], mx)));
    for (uint32_t j = 0; j < k; ++j) {
        uint32_t best = 0;
        float bs = -FLT_MAX;
        for (uint32_t q = 0; q < experts; ++q) {
            if (scratch[q] > bs) {
                bs = scratch[q];
                best = q;
            }
        }
        idx[size_t(tok) * k + j] = best;
        scratch[best] = -FLT_MAX;
    }
    for (uint32_t j = 0; j < k; ++j)
        weights[size_t(tok) * k + j] = fdiv(expf(__fsub_rn(s[idx[size_t(tok) * k + j]], mx)), sum);
}

// vyre-libs/src/nn/moe/topk_selection.rs:23-92 on the global best_vals/best_idxs slots
__device__ void topk_insert(float* vals, uint32_t* idxs, uint32_t k, float v, uint32_t i) {
    uint32_t pos = k;
    for (uint32_t j = 0; j < k; ++j)
        if (pos == k && v > vals[j]) pos = j;
    if (pos < k) {
        for (uint32_t rev = k - 1; rev > pos; --rev) {
            vals[rev] = vals[rev - 1];
            idxs[rev] = idxs[rev - 1];
        }
        vals[pos] = v;
        idxs[pos] = i;
    }
}
__global__ void softmax_top_k_kernel(const float* scores, uint32_t* out_idx, float* out_w, float* vals,
                                     uint32_t* idxs, uint32_t n, uint32_t k) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    for (uint32_t s = 0; s < k; ++s) {
        vals[s] = -INFINITY;
        idxs[s] = 0;
    }
    float mx = -INFINITY;
    for (uint32_t i = 0; i < n; ++i)
        if (scores[i] > mx) mx = scores[i];
    float sum = 0.0f;
    for (uint32_t i = 0; i < n; ++i) {
        const float e = expf(__fsub_rn(scores[i], mx));
        sum = fadd(sum, e);
        topk_insert(vals, idxs, k, e, i);
    }
    for (uint32_t s = 0; s < k; ++s) {
        out_w[s] = fdiv(vals[s], sum);
        out_idx[s] = idxs[s];
    }
}
__global__ void top_k_kernel(const float* in, uint32_t* out_idx, float* vals, uint32_t* idxs, uint32_t n, uint32_t k) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    for (uint32_t s = 0; s < k; ++s) {
        vals[s] = -INFINITY;
        idxs[s] = 0;
    }
    for (uint32_t i = 0; i < n; ++i) topk_insert(vals, idxs, k, in[i], i);
    for (uint32_t s = 0; s < k; ++s) out_idx[s] = idxs[s];
}

// vyre-libs/src/nn/activation/unary.rs:79-100: gate * (up * (1/(1+exp(-gate))))
__global__ void swiglu_kernel(const void* gate, const void* up, void* out, uint32_t n, uint32_t dt) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = load_typed(gate, i, dt), u = load_typed(up, i, dt);
    const float sig = fdiv(1.0f, fadd(1.0f, expf(-g)));
    store_typed(out, i, dt, fmul(g, fmul(u, sig)));
}

// vyre-libs/src/nn/activation/residual_add.rs:40-52: cast(dtype, f32(residual) + f32(branch))
__global__ void residual_add_kernel(const void* residual, const void* branch, void* out, uint32_t n, uint32_t dt) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    store_typed(out, i, dt, fadd(load_typed(residual, i, dt), load_typed(branch, i, dt)));
}

// vyre-libs/src/nn/norm/gated_rms_norm.rs:123-247. The reference recomputes the row's sum of squares in every
// invocation, one f32 chain over the row in index order; here one block owns a row: its threads stage the row through
// shared memory (coalesced), thread 0 runs that same chain once, and all threads then normalise (x * (1 / sqrt(mean +
// eps)), rounded to dtype, times f32(weight), times gate / (1 + exp(-gate)) with a gate, one cast). Same values.
__global__ void rms_norm_kernel(const void* input, const void* weight, const void* gate, void* out, uint32_t hidden, float eps,
                                uint32_t dt, uint32_t wdt) {
    __shared__ float tile[1024];
    __shared__ float inv_shared;
    const size_t base = size_t(blockIdx.x) * hidden;
    float sum = 0.0f;
    for (uint32_t c0 = 0; c0 < hidden; c0 += 1024) {
        const uint32_t len = min(1024u, hidden - c0);
        for (uint32_t c = threadIdx.x; c < len; c += blockDim.x) {
            const float v = load_typed(input, base + c0 + c, dt);
            tile[c] = fmul(v, v);
        }
        __syncthreads();
        if (threadIdx.x == 0)
            for (uint32_t c = 0; c < len; ++c) sum = fadd(sum, tile[c]);
        __syncthreads();
    }
    if (threadIdx.x == 0) inv_shared = fdiv(1.0f, __fsqrt_rn(fadd(fdiv(sum, float(hidden)), eps)));
    __syncthreads();
    const float inv = inv_shared;
    for (uint32_t c = threadIdx.x; c < hidden; c += blockDim.x) {
        float normalized = fmul(load_typed(input, base + c, dt), inv);
        if (dt == 1) normalized = __bfloat162float(__float2bfloat16_rn(normalized));
        else if (dt == 2) normalized = __half2float(__float2half_rn(normalized));
        float v = fmul(normalized, load_typed(weight, c, wdt));
        if (gate) {
            const float g = load_typed(gate, base + c, dt);
            v = fmul(v, fdiv(g, fadd(1.0f, expf(-g))));
        }
        store_typed(out, base + c, dt, v);
    }
}

// The same operator for long rows: the row's sum of squares as a two-level tree (every thread a strided partial sum,
// warp shuffles, eight warp sums added in warp order) instead of one chain of `hidden` dependent additions, which at
// hidden = 4096 is 8 microseconds on one thread. Deterministic; differs from the chain by f32 rounding of the sum
// (about 1e-7 relative), everything after the sum is the code above.
__global__ void __launch_bounds__(256) rms_norm_tree_kernel(const void* input, const void* weight, const void* gate, void* out,
                                                            uint32_t hidden, float eps, uint32_t dt, uint32_t wdt) {
    __shared__ float warp_sum[8];
    __shared__ float inv_shared;
    const size_t base = size_t(blockIdx.x) * hidden;
    float sum = 0.0f;
    for (uint32_t c = threadIdx.x; c < hidden; c += 256) {
        const float v = load_typed(input, base + c, dt);
        sum = fadd(sum, fmul(v, v));
    }
    for (int o = 16; o > 0; o >>= 1) sum = fadd(sum, __shfl_xor_sync(0xffffffffu, sum, o));
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < 8; ++w) total = fadd(total, warp_sum[w]);
        inv_shared = fdiv(1.0f, __fsqrt_rn(fadd(fdiv(total, float(hidden)), eps)));
    }
    __syncthreads();
    const float inv = inv_shared;
    for (uint32_t c = threadIdx.x; c < hidden; c += 256) {
        float normalized = fmul(load_typed(input, base + c, dt), inv);
        if (dt == 1) normalized = __bfloat162float(__float2bfloat16_rn(normalized));
        else if (dt == 2) normalized = __half2float(__float2half_rn(normalized));
        float v = fmul(normalized, load_typed(weight, c, wdt));
        if (gate) {
            const float g = load_typed(gate, base + c, dt);
            v = fmul(v, fdiv(g, fadd(1.0f, expf(-g))));
        }
        store_typed(out, base + c, dt, v);
    }
}

// vyre-libs/src/nn/quant/ggml.rs:28-120 and 217-333. bits = 4: blocks of 32 weights in 4 words; bits = 2: blocks of 16 in 1
__device__ __forceinline__ uint32_t k_quant_value(const uint32_t* packed, uint32_t linear, uint32_t bits, uint32_t* block) {
    const uint32_t block_size = bits == 4 ? 32u : 16u, values_per_byte = 8u / bits, words_per_block = bits == 4 ? 4u : 1u;
    const uint32_t block_idx = linear / block_size, within = linear % block_size;
    const uint32_t byte_idx = within / values_per_byte, value_shift = (within % values_per_byte) * bits;
    const uint32_t word = packed[size_t(block_idx) * words_per_block + byte_idx / 4];
    *block = block_idx;
    return (word >> ((byte_idx % 4) * 8 + value_shift)) & ((1u << bits) - 1u);
}
__global__ void k_quant_unpack_kernel(const uint32_t* packed, const float* scales, const float* mins, float* out, uint32_t n,
                                      uint32_t bits) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t block;
    const uint32_t q = k_quant_value(packed, i, bits, &block);
    out[i] = fadd(fmul(float(q), scales[block]), mins[block]);
}
// thread per output, k ascending, every product and sum rounded on its own. Neighbouring outputs sit in neighbouring
// nibbles of the k-major weight stream, so a warp reads 16 (Q4_K) or 8 (Q2_K) contiguous bytes per k.
__global__ void k_quant_linear_kernel(const float* x, const uint32_t* packed, const float* scales, const float* mins,
                                      const float* b, float* out, uint32_t in_dim, uint32_t out_dim, uint32_t bits) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= out_dim) return;
    float acc = b[i];
    for (uint32_t k = 0; k < in_dim; ++k) {
        uint32_t block;
        const uint32_t q = k_quant_value(packed, k * out_dim + i, bits, &block);
        const float weight = fadd(fmul(float(q), scales[block]), mins[block]);
        acc = fadd(acc, fmul(x[k], weight));
    }
    out[i] = acc;
}

// vyre-libs/src/nn/moe/expert_mlp.rs:46-150 split in two launches: hidden activations once, then the down
// projection (the reference recomputes the hidden vector per output thread; values are identical).
__global__ void expert_hidden_kernel(const float* x, const float* wg, const float* bg, const float* wu,
                                     const float* bu, float* hid, uint32_t in_dim, uint32_t hidden) {
    const uint32_t h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h >= hidden) return;
    float g = bg[h], u = bu[h];
    for (uint32_t k = 0; k < in_dim; ++k) {
        g = fadd(g, fmul(x[k], wg[size_t(k) * hidden + h]));
        u = fadd(u, fmul(x[k], wu[size_t(k) * hidden + h]));
    }
    const float sig = fdiv(1.0f, fadd(1.0f, expf(-g)));
    hid[h] = fmul(fmul(g, sig), u);
}
__global__ void expert_down_kernel(const float* hid, const float* wd, const float* bd, float* out, uint32_t hidden,
                                   uint32_t out_dim) {
    const uint32_t o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= out_dim) return;
    float acc = bd[o];
    for (uint32_t h = 0; h < hidden; ++h) acc = fadd(acc, fmul(hid[h], wd[size_t(h) * out_dim + o]));
    out[o] = acc;
}

// vyre-libs/src/nn/moe/moe_layer.rs:57-101
__global__ void moe_accumulate_kernel(const float* weights, const float* expert_out, float* out, uint32_t k,
                                      uint32_t out_dim) {
    const uint32_t j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= out_dim) return;
    float acc = 0.0f;
    for (uint32_t e = 0; e < k; ++e) acc = fadd(acc, fmul(weights[e], expert_out[size_t(e) * out_dim + j]));
    out[j] = acc;
}

inline uint32_t blocks(uint64_t n, uint32_t per) { return uint32_t((n + per - 1) / per); }

}  // namespace

cudaError_t launch_linear_4bit(const float* x, const uint32_t* w, const float* b, float* out, uint32_t in_dim,
                               uint32_t out_dim, cudaStream_t s) {
    linear_4bit_kernel<<<blocks(out_dim, 256), 256, 0, s>>>(x, w, b, out, in_dim, out_dim);
    return cudaGetLastError();
}
cudaError_t launch_linear_4bit_affine_grouped(const float* x, const uint32_t* w, const float* scale,
                                              const uint32_t* zp, const float* b, float* out, uint32_t in_dim,
                                              uint32_t out_dim, uint32_t group, uint32_t batch, cudaStream_t s) {
    const uint32_t total = batch * out_dim;
    affine_grouped_kernel<<<blocks(total, 8), 256, 0, s>>>(x, w, scale, zp, b, out, in_dim, out_dim, group, total);
    return cudaGetLastError();
}
cudaError_t launch_i4_unpack(const uint32_t* packed, int32_t* out, uint32_t lanes, cudaStream_t s) {
    i4_unpack_kernel<<<blocks(lanes, 256), 256, 0, s>>>(packed, out, lanes);
    return cudaGetLastError();
}
cudaError_t launch_i4_dot_i32(const uint32_t* lhs, const uint32_t* rhs, int32_t* out, uint32_t lanes, cudaStream_t s) {
    i4_dot_i32_kernel<<<1, 1, 0, s>>>(lhs, rhs, out, lanes);
    return cudaGetLastError();
}
cudaError_t launch_i4_dot_f32_scaled(const uint32_t* lhs, const uint32_t* rhs, const float* ls, const float* rs,
                                     float* out, uint32_t lanes, cudaStream_t s) {
    i4_dot_f32_scaled_kernel<<<1, 1, 0, s>>>(lhs, rhs, ls, rs, out, lanes);
    return cudaGetLastError();
}
cudaError_t launch_i4_batched_matvec(const uint32_t* w, const float* x, const float* scales, float* out,
                                     uint32_t batch, uint32_t rows, uint32_t cols, cudaStream_t s) {
    i4_batched_matvec_kernel<<<blocks(uint64_t(batch) * rows, 64), 64, 0, s>>>(w, x, scales, out, batch, rows, cols);
    return cudaGetLastError();
}
cudaError_t launch_i4_batched_matmul(const uint32_t* w, const uint32_t* act, const float* rs, const float* bs,
                                     float* out, uint32_t batch, uint32_t rows, uint32_t cols, cudaStream_t s) {
    i4_batched_matmul_kernel<<<blocks(uint64_t(batch) * rows, 64), 64, 0, s>>>(w, act, rs, bs, out, batch, rows, cols);
    return cudaGetLastError();
}
cudaError_t launch_i4_batched_matmul_top1(const uint32_t* w, const uint32_t* act, const float* rs, const float* bs,
                                          float* out, uint32_t batch, uint32_t rows, uint32_t cols, cudaStream_t s) {
    i4_batched_matmul_top1_kernel<<<blocks(batch, 64), 64, 0, s>>>(w, act, rs, bs, out, batch, rows, cols);
    return cudaGetLastError();
}
cudaError_t launch_int8_unpack(const uint32_t* packed, const float* scales, float* out, uint32_t n, uint32_t cols,
                               cudaStream_t s) {
    int8_unpack_kernel<<<blocks(n, 64), 64, 0, s>>>(packed, scales, out, n, cols);
    return cudaGetLastError();
}
cudaError_t launch_int8_pack(const uint32_t* in, uint32_t* out, uint32_t n, cudaStream_t s) {
    int8_pack_kernel<<<blocks(n, 64), 64, 0, s>>>(in, out, n);
    return cudaGetLastError();
}
cudaError_t launch_linear_rows(const void* x, const void* w, const void* bias, void* out, uint32_t rows,
                               uint32_t in_dim, uint32_t out_dim, uint32_t dtype, uint32_t out_in, cudaStream_t s) {
    linear_rows_kernel<<<blocks(uint64_t(rows) * out_dim, 64), 64, 0, s>>>(x, w, bias, out, rows, in_dim, out_dim,
                                                                           dtype, out_in);
    return cudaGetLastError();
}
cudaError_t launch_matmul_u32(const uint32_t* a, const uint32_t* b, const uint32_t* bias, uint32_t* out, uint32_t m,
                              uint32_t k, uint32_t n, cudaStream_t s) {
    const uint32_t gy = (m + 31) / 32;
    if (gy > 65535u) return cudaErrorInvalidValue;
    matmul_u32_kernel<<<dim3((n + 31) / 32, gy), 256, 0, s>>>(a, b, bias, out, m, k, n);
    return cudaGetLastError();
}
cudaError_t launch_moe_gate(const float* scores, uint32_t* idx, float* weights, uint32_t tokens, uint32_t experts,
                            uint32_t k, cudaStream_t s) {
    // threads per block limited so that the per-thread expert scratch fits the default 48 KB of shared memory
    uint32_t tpb = 128;
    while (tpb > 1 && size_t(tpb) * experts * 4 > 48 * 1024) tpb >>= 1;
    if (size_t(tpb) * experts * 4 > 48 * 1024) return cudaErrorInvalidValue;
    moe_gate_kernel<<<blocks(tokens, tpb), tpb, size_t(tpb) * experts * 4, s>>>(scores, idx, weights, tokens, experts, k);
    return cudaGetLastError();
}
cudaError_t launch_softmax_top_k(const float* scores, uint32_t* out_idx, float* out_w, float* best_vals,
                                 uint32_t* best_idxs, uint32_t n, uint32_t k, cudaStream_t s) {
    softmax_top_k_kernel<<<1, 1, 0, s>>>(scores, out_idx, out_w, best_vals, best_idxs, n, k);
    return cudaGetLastError();
}
cudaError_t launch_top_k(const float* in, uint32_t* out_idx, float* best_vals, uint32_t* best_idxs, uint32_t n,
                         uint32_t k, cudaStream_t s) {
    top_k_kernel<<<1, 1, 0, s>>>(in, out_idx, best_vals, best_idxs, n, k);
    return cudaGetLastError();
}
cudaError_t launch_residual_add(const void* residual, const void* branch, void* out, uint32_t n, uint32_t dtype, cudaStream_t s) {
    residual_add_kernel<<<blocks(n, 256), 256, 0, s>>>(residual, branch, out, n, dtype);
    return cudaGetLastError();
}
cudaError_t launch_rms_norm(const void* input, const void* weight, const void* gate, void* out, uint32_t rows, uint32_t hidden,
                            float eps, uint32_t dtype, uint32_t weight_dtype, bool tree, cudaStream_t s) {
    if (tree) rms_norm_tree_kernel<<<rows, 256, 0, s>>>(input, weight, gate, out, hidden, eps, dtype, weight_dtype);
    else rms_norm_kernel<<<rows, 256, 0, s>>>(input, weight, gate, out, hidden, eps, dtype, weight_dtype);
    return cudaGetLastError();
}
cudaError_t launch_k_quant_unpack(const uint32_t* packed, const float* scales, const float* mins, float* out, uint32_t n,
                                  uint32_t bits, cudaStream_t s) {
    k_quant_unpack_kernel<<<blocks(n, 256), 256, 0, s>>>(packed, scales, mins, out, n, bits);
    return cudaGetLastError();
}
cudaError_t launch_k_quant_linear(const float* x, const uint32_t* packed, const float* scales, const float* mins, const float* b,
                                  float* out, uint32_t in_dim, uint32_t out_dim, uint32_t bits, cudaStream_t s) {
    k_quant_linear_kernel<<<blocks(out_dim, 64), 64, 0, s>>>(x, packed, scales, mins, b, out, in_dim, out_dim, bits);
    return cudaGetLastError();
}
cudaError_t launch_swiglu(const void* gate, const void* up, void* out, uint32_t n, uint32_t dtype, cudaStream_t s) {
    swiglu_kernel<<<blocks(n, 256), 256, 0, s>>>(gate, up, out, n, dtype);
    return cudaGetLastError();
}
cudaError_t launch_expert_mlp(const float* x, const float* wg, const float* bg, const float* wu, const float* bu,
                              const float* wd, const float* bd, float* out, float* hidden_scratch, uint32_t in_dim,
                              uint32_t hidden, uint32_t out_dim, cudaStream_t s) {
    expert_hidden_kernel<<<blocks(hidden, 64), 64, 0, s>>>(x, wg, bg, wu, bu, hidden_scratch, in_dim, hidden);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    expert_down_kernel<<<blocks(out_dim, 64), 64, 0, s>>>(hidden_scratch, wd, bd, out, hidden, out_dim);
    return cudaGetLastError();
}
cudaError_t launch_moe_layer_accumulate(const float* weights, const float* expert_out, float* out, uint32_t k,
                                        uint32_t out_dim, cudaStream_t s) {
    moe_accumulate_kernel<<<blocks(out_dim, 256), 256, 0, s>>>(weights, expert_out, out, k, out_dim);
    return cudaGetLastError();
}

}  // namespace vybk
