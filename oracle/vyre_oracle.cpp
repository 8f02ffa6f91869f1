// TEST INFRASTRUCTURE ONLY - CPU restatement of vyre's reference-engine semantics for the
// quantized-linear / MoE hot path. Nothing in the product library links or calls this file;
// it is the checker used by the tests, by the smoke run and by the benchmark's CPU-baseline leg.
//
// Every function cites the reference source (paths relative to the vyre tree) whose
// semantics it restates. The reference is Rust and cannot be compiled in this environment,
// so the restatement is pinned against the reference's own golden vectors (see
// tests/test_oracle_golden.py). The one third-party dependency on the path is the `libm`
// crate (pinned =0.2.16, vyre-reference/src/ieee754.rs:89-91, `canonical_exp -> libm::expf`);
// here `expf` comes from glibc and is compared under the reference's own 128-ULP
// transcendental window (vyre-foundation/src/fp_parity.rs:14-16).
//
// Build: g++ -O2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
// -ffp-contract=off is load-bearing: the reference distinguishes a*b+c (two roundings)
// from Fma (one rounding).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#include <algorithm>
#include <limits>

#ifdef _OPENMP
#include <omp.h>
#endif

#define VYO_API extern "C" __attribute__((visibility("default")))

namespace {

// vyre-reference/src/execution/typed_ops/float_ops.rs:82-90: NaN -> 0x7FC00000,
// subnormal -> signed zero; applied to operands and results of every f32 op.
inline float canon(float v) {
    uint32_t b;
    std::memcpy(&b, &v, 4);
    if ((b & 0x7f800000u) == 0x7f800000u && (b & 0x007fffffu) != 0) {
        b = 0x7fc00000u;
    } else if ((b & 0x7f800000u) == 0 && (b & 0x007fffffu) != 0) {
        b &= 0x80000000u;
    }
    float r;
    std::memcpy(&r, &b, 4);
    return r;
}
inline float f_add(float a, float b) { return canon(canon(a) + canon(b)); }
inline float f_sub(float a, float b) { return canon(canon(a) - canon(b)); }
inline float f_mul(float a, float b) { return canon(canon(a) * canon(b)); }
inline float f_div(float a, float b) { return canon(canon(a) / canon(b)); }
inline float f_neg(float a) { return canon(-canon(a)); }
// vyre-reference/src/execution/expr.rs:237-275: Fma = single-rounding mul_add, then canonicalise.
inline float f_fma(float a, float b, float c) { return canon(std::fmaf(canon(a), canon(b), canon(c))); }
// vyre-reference/src/ieee754.rs:89-91 (libm::expf in the reference, glibc here).
inline float f_exp(float a) { return canon(std::exp(canon(a))); }
inline float f_max(float a, float b) { return canon(std::fmax(canon(a), canon(b))); }

// vyre-reference/src/float16.rs:5-16
inline float bf16_to_f32(uint16_t bits) {
    uint32_t b = uint32_t(bits) << 16;
    float r;
    std::memcpy(&r, &b, 4);
    return canon(r);
}
inline uint16_t f32_to_bf16(float value) {
    float c = canon(value);
    uint32_t bits;
    std::memcpy(&bits, &c, 4);
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x007fffffu) != 0) return 0x7fc0;
    uint32_t rounded = bits + (0x7fffu + ((bits >> 16) & 1u));
    return uint16_t(rounded >> 16);
}
// vyre-reference/src/float16.rs:18-87
inline float f16_to_f32(uint16_t bits) {
    uint32_t sign = uint32_t(bits & 0x8000u) << 16;
    uint32_t exponent = (bits >> 10) & 0x1f;
    uint32_t fraction = bits & 0x03ff;
    uint32_t result;
    if (exponent == 0 && fraction == 0) {
        result = sign;
    } else if (exponent == 0) {
        uint32_t leading = 31 - uint32_t(__builtin_clz(fraction));
        uint32_t shift = 10 - leading;
        uint32_t nf = (fraction << shift) & 0x03ff;
        int32_t unbiased = -14 - int32_t(shift);
        result = sign | (uint32_t(unbiased + 127) << 23) | (nf << 13);
    } else if (exponent == 0x1f && fraction == 0) {
        result = sign | 0x7f800000u;
    } else if (exponent == 0x1f) {
        result = 0x7fc00000u;
    } else {
        result = sign | ((exponent + 112) << 23) | (fraction << 13);
    }
    float r;
    std::memcpy(&r, &result, 4);
    return canon(r);
}
inline uint32_t round_shift_right(uint32_t value, uint32_t shift) {
    if (shift == 0) return value;
    uint32_t q = value >> shift;
    uint32_t mask = (1u << shift) - 1;
    uint32_t rem = value & mask;
    uint32_t half = 1u << (shift - 1);
    return q + uint32_t(rem > half || (rem == half && (q & 1u) == 1u));
}
inline uint16_t f32_to_f16(float value) {
    float c = canon(value);
    uint32_t bits;
    std::memcpy(&bits, &c, 4);
    uint16_t sign = uint16_t((bits >> 16) & 0x8000u);
    int32_t exponent = int32_t((bits >> 23) & 0xff);
    uint32_t fraction = bits & 0x007fffffu;
    if (exponent == 0xff) return fraction == 0 ? uint16_t(sign | 0x7c00) : uint16_t(0x7e00);
    if (exponent == 0) return sign;
    int32_t unbiased = exponent - 127;
    if (unbiased > 15) return uint16_t(sign | 0x7c00);
    if (unbiased >= -14) {
        uint16_t he = uint16_t(unbiased + 15);
        uint32_t rf = round_shift_right(fraction, 13);
        if (rf == 0x400) {
            he = uint16_t(he + 1);
            if (he >= 0x1f) return uint16_t(sign | 0x7c00);
            return uint16_t(sign | (he << 10));
        }
        return uint16_t(sign | (he << 10) | uint16_t(rf));
    }
    if (unbiased < -25) return sign;
    uint32_t significand = 0x00800000u | fraction;
    uint32_t shift = uint32_t(-unbiased - 1);
    uint32_t rounded = round_shift_right(significand, shift);
    if (rounded >= 0x400) return uint16_t(sign | 0x0400);
    return uint16_t(sign | uint16_t(rounded));
}

// dtype tags follow vyre-spec/src/data_type.rs (F16, BF16, F32 only matter here).
enum : uint32_t { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };

inline float load_typed(const void* p, size_t i, uint32_t dt) {
    switch (dt) {
        case DT_BF16: return bf16_to_f32(static_cast<const uint16_t*>(p)[i]);
        case DT_F16: return f16_to_f32(static_cast<const uint16_t*>(p)[i]);
        default: return canon(static_cast<const float*>(p)[i]);
    }
}
inline void store_typed(void* p, size_t i, uint32_t dt, float v) {
    switch (dt) {
        case DT_BF16: static_cast<uint16_t*>(p)[i] = f32_to_bf16(v); break;
        case DT_F16: static_cast<uint16_t*>(p)[i] = f32_to_f16(v); break;
        default: static_cast<float*>(p)[i] = canon(v); break;
    }
}

// vyre-primitives/src/math/quantized/cpu.rs:262-274 (extract_i4_lane): out-of-range word reads 0.
inline int32_t extract_i4_lane(const uint32_t* packed, size_t words, size_t lane) {
    size_t wi = lane / 8;
    uint32_t word = wi < words ? packed[wi] : 0u;
    uint32_t shift = uint32_t(lane % 8) * 4;
    int32_t nib = int32_t((word >> shift) & 0xF);
    return (nib & 0x8) == 0 ? nib : nib - 16;
}
inline size_t i4_words(size_t lanes) { return (lanes + 7) / 8; }

}  // namespace

// ---------------------------------------------------------------------------------------------
// scalar helpers exported for the pin tests
// ---------------------------------------------------------------------------------------------
VYO_API float vyo_canonical_f32(float v) { return canon(v); }
VYO_API float vyo_bf16_to_f32(uint16_t b) { return bf16_to_f32(b); }
VYO_API uint16_t vyo_f32_to_bf16(float v) { return f32_to_bf16(v); }
VYO_API float vyo_f16_to_f32(uint16_t b) { return f16_to_f32(b); }
VYO_API uint16_t vyo_f32_to_f16(float v) { return f32_to_f16(v); }

// vyre-reference/src/ieee754.rs:170-205 (canonical_ulp_distance)
VYO_API uint32_t vyo_ulp_distance(float a, float b) {
    float l = canon(a), r = canon(b);
    uint32_t lb, rb;
    std::memcpy(&lb, &l, 4);
    std::memcpy(&rb, &r, 4);
    if (l == r || lb == rb) return 0;
    auto key = [](uint32_t bits) { return (bits & 0x80000000u) == 0 ? (bits | 0x80000000u) : ~bits; };
    uint32_t kl = key(lb), kr = key(rb);
    return kl > kr ? kl - kr : kr - kl;
}

// ---------------------------------------------------------------------------------------------
// packed INT4 primitives - vyre-primitives/src/math/quantized/cpu.rs
// ---------------------------------------------------------------------------------------------
// cpu.rs:35-61 try_pack_i4x8_cpu_into: clamp to [-8,7], two's-complement nibble, lane i%8 at bit 4(i%8).
VYO_API void vyo_pack_i4x8(const int32_t* values, uint32_t lanes, uint32_t* out_words) {
    size_t words = i4_words(lanes);
    for (size_t w = 0; w < words; ++w) out_words[w] = 0;
    for (uint32_t i = 0; i < lanes; ++i) {
        int32_t c = std::min(7, std::max(-8, values[i]));
        uint32_t nib = uint32_t(uint8_t(int8_t(c))) & 0x0Fu;
        out_words[i / 8] |= nib << ((i % 8) * 4);
    }
}
// cpu.rs:64-104
VYO_API void vyo_unpack_i4x8(const uint32_t* packed, uint32_t words, uint32_t lanes, int32_t* out) {
    for (uint32_t i = 0; i < lanes; ++i) out[i] = extract_i4_lane(packed, words, i);
}
// cpu.rs:108-118 (wrapping i32)
VYO_API int32_t vyo_i4x8_dot_i32(const uint32_t* lhs, const uint32_t* rhs, uint32_t lanes) {
    size_t words = i4_words(lanes);
    uint32_t acc = 0;
    for (uint32_t i = 0; i < lanes; ++i) {
        uint32_t l = uint32_t(extract_i4_lane(lhs, words, i));
        uint32_t r = uint32_t(extract_i4_lane(rhs, words, i));
        acc += l * r;
    }
    return int32_t(acc);
}
// cpu.rs:122-137: acc += lhs*rhs (two roundings), then acc*lhs_scale*rhs_scale.
VYO_API float vyo_i4x8_dot_f32_scaled(const uint32_t* lhs, const uint32_t* rhs, float ls, float rs,
                                      uint32_t lanes) {
    size_t words = i4_words(lanes);
    float acc = 0.0f;
    for (uint32_t i = 0; i < lanes; ++i) {
        float l = float(extract_i4_lane(lhs, words, i));
        float r = float(extract_i4_lane(rhs, words, i));
        acc = f_add(acc, f_mul(l, r));
    }
    return f_mul(f_mul(acc, ls), rs);
}
// cpu.rs:141-163 and program_helpers.rs:7-81: per row sequential acc += w*x, then acc*scale[row].
VYO_API void vyo_i4x8_batched_matvec_f32_scaled(const uint32_t* w, const float* x, const float* scales,
                                                uint32_t batch, uint32_t rows, uint32_t cols, float* out) {
    size_t wpr = i4_words(cols);
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t b = 0; b < batch; ++b) {
        for (uint32_t r = 0; r < rows; ++r) {
            const uint32_t* wr = w + size_t(r) * wpr;
            const float* xb = x + size_t(b) * cols;
            float acc = 0.0f;
            for (uint32_t c = 0; c < cols; ++c)
                acc = f_add(acc, f_mul(float(extract_i4_lane(wr, wpr, c)), xb[c]));
            out[size_t(b) * rows + r] = f_mul(acc, scales[r]);
        }
    }
}
VYO_API void vyo_i4x8_matvec_f32_scaled(const uint32_t* w, const float* x, const float* scales,
                                        uint32_t rows, uint32_t cols, float* out) {
    vyo_i4x8_batched_matvec_f32_scaled(w, x, scales, 1, rows, cols, out);
}
// cpu.rs:195-222: int4 x int4, acc*row_scale*batch_scale.
VYO_API void vyo_i4x8_batched_matmul_f32_scaled(const uint32_t* w, const uint32_t* act, const float* row_scales,
                                                const float* batch_scales, uint32_t batch, uint32_t rows,
                                                uint32_t cols, float* out) {
    size_t wpr = i4_words(cols);
    for (uint32_t b = 0; b < batch; ++b) {
        const uint32_t* ab = act + size_t(b) * wpr;
        for (uint32_t r = 0; r < rows; ++r) {
            const uint32_t* wr = w + size_t(r) * wpr;
            float acc = 0.0f;
            for (uint32_t c = 0; c < cols; ++c)
                acc = f_add(acc, f_mul(float(extract_i4_lane(wr, wpr, c)), float(extract_i4_lane(ab, wpr, c))));
            out[size_t(b) * rows + r] = f_mul(f_mul(acc, row_scales[r]), batch_scales[b]);
        }
    }
}
// cpu.rs:227-259: strict '>' argmax, first max wins, init f32::MIN; out = [scores(batch) || f32(index)(batch)]
// (output layout: vyre-primitives/src/math/quantized/programs.rs:457-616).
VYO_API void vyo_i4x8_batched_matmul_top1_f32_scaled(const uint32_t* w, const uint32_t* act,
                                                     const float* row_scales, const float* batch_scales,
                                                     uint32_t batch, uint32_t rows, uint32_t cols, float* out) {
    std::vector<float> logits(size_t(batch) * rows);
    vyo_i4x8_batched_matmul_f32_scaled(w, act, row_scales, batch_scales, batch, rows, cols, logits.data());
    for (uint32_t b = 0; b < batch; ++b) {
        float best = std::numeric_limits<float>::lowest();
        uint32_t idx = 0;
        for (uint32_t r = 0; r < rows; ++r) {
            float s = logits[size_t(b) * rows + r];
            if (s > best) { best = s; idx = r; }
        }
        out[b] = best;
        out[batch + b] = float(idx);
    }
}

// ---------------------------------------------------------------------------------------------
// vyre-libs::nn::linear_4bit - vyre-libs/src/nn/linear/inner/linear_4bit.rs:255-335
// out[i] = b[i] + sum_k x[k]*f32(nib(k,i)), sequential k, mul then add.
// ---------------------------------------------------------------------------------------------
VYO_API void vyo_linear_4bit(const float* x, const uint32_t* w, const float* b, float* out,
                             uint32_t in_dim, uint32_t out_dim) {
#pragma omp parallel for schedule(static)
    for (uint32_t i = 0; i < out_dim; ++i) {
        float acc = canon(b[i]);
        for (uint32_t k = 0; k < in_dim; ++k) {
            uint32_t word = w[size_t(k / 8) * out_dim + i];
            float nib = float((word >> ((k % 8) * 4)) & 0xFu);
            acc = f_add(acc, f_mul(x[k], nib));
        }
        out[i] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// vyre-libs::nn::linear_4bit_affine_grouped (+ batched, + weight-reuse variant) in the reference
// interpreter's evaluation order - linear_4bit.rs:505-708 (lane l accumulates k = 32c + l with
// acc = fma(x, fma(f32(nib), s, fma(f32(zp), fma(-1, s, -0), -0)), acc)), then the subgroup fold
// lanes 0..31 from 0.0 (vyre-reference/src/execution/hashmap/subgroup.rs:87-117), then b[i] + sum.
// The weight-reuse variant (linear_4bit.rs:778-997) stages the same fma-dequantised weight and
// accumulates in the same lane order, so one routine covers all variants.
// Layout: w[(k/8)*out_dim + i], nibble k%8 at bit 4(k%8); sidecars [group][out_dim].
// ---------------------------------------------------------------------------------------------
VYO_API void vyo_linear_4bit_affine_grouped(const float* x, const uint32_t* w, const float* scale,
                                            const uint32_t* zp, const float* b, float* out, uint32_t in_dim,
                                            uint32_t out_dim, uint32_t group_size, uint32_t batch) {
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t bi = 0; bi < batch; ++bi) {
        for (uint32_t i = 0; i < out_dim; ++i) {
            const float* xb = x + size_t(bi) * in_dim;
            float lane_acc[32];
            for (uint32_t lane = 0; lane < 32; ++lane) {
                float acc = 0.0f;
                for (uint32_t k = lane; k < in_dim; k += 32) {
                    uint32_t word = w[size_t(k / 8) * out_dim + i];
                    float nib = float((word >> ((k % 8) * 4)) & 0xFu);
                    size_t side = size_t(k / group_size) * out_dim + i;
                    float s = scale[side];
                    float neg_s = f_fma(-1.0f, s, -0.0f);
                    float zero_off = f_fma(float(zp[side]), neg_s, -0.0f);
                    float wv = f_fma(nib, s, zero_off);
                    acc = f_fma(xb[k], wv, acc);
                }
                lane_acc[lane] = acc;
            }
            float sum = 0.0f;
            for (uint32_t lane = 0; lane < 32; ++lane) sum = f_add(sum, lane_acc[lane]);
            out[size_t(bi) * out_dim + i] = f_add(b[i], sum);
        }
    }
}

// The reference's own hand loop used as expected value in its tests and as its benchmark's CPU baseline:
// acc = bias; acc += x[k] * (nib - zp) * scale  (linear_4bit.rs:1186-1208; vyre-bench/src/cases/quantized_linear.rs:447-463).
VYO_API void vyo_linear_4bit_affine_grouped_simple(const float* x, const uint32_t* w, const float* scale,
                                                   const uint32_t* zp, const float* b, float* out,
                                                   uint32_t in_dim, uint32_t out_dim, uint32_t group_size,
                                                   uint32_t batch) {
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t bi = 0; bi < batch; ++bi) {
        for (uint32_t i = 0; i < out_dim; ++i) {
            const float* xb = x + size_t(bi) * in_dim;
            float acc = b[i];
            for (uint32_t k = 0; k < in_dim; ++k) {
                uint32_t word = w[size_t(k / 8) * out_dim + i];
                float nib = float((word >> ((k % 8) * 4)) & 0xFu);
                size_t side = size_t(k / group_size) * out_dim + i;
                float t = xb[k] * (nib - float(zp[side]));
                acc += t * scale[side];
            }
            out[size_t(bi) * out_dim + i] = acc;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// int8 pack/unpack - vyre-libs/src/nn/quant/int8.rs:15-78 (one value per u32 word, unsigned cast)
// ---------------------------------------------------------------------------------------------
VYO_API void vyo_int8_unpack(const uint32_t* packed, const float* scales, float* out, uint32_t n, uint32_t cols) {
    for (uint32_t i = 0; i < n; ++i) out[i] = f_mul(float(packed[i]), scales[i / cols]);
}
VYO_API void vyo_int8_pack(const uint32_t* in, uint32_t* out, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i) out[i] = in[i] & 0xFFu;
}

// ---------------------------------------------------------------------------------------------
// linear_rows family - vyre-libs/src/nn/linear/inner/builder.rs:253-361
// out[r,c] = cast(dtype, bias?[c] + sum_k f32(x[r,k])*f32(w[idx])), sequential k, mul then add;
// weight_out_in ? w[c*in+k] : w[k*out+c].
// ---------------------------------------------------------------------------------------------
VYO_API void vyo_linear_rows(const void* x, const void* w, const void* bias, void* out, uint32_t rows,
                             uint32_t in_dim, uint32_t out_dim, uint32_t dtype, uint32_t weight_out_in) {
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t r = 0; r < rows; ++r) {
        for (uint32_t c = 0; c < out_dim; ++c) {
            float acc = bias ? load_typed(bias, c, dtype) : 0.0f;
            for (uint32_t k = 0; k < in_dim; ++k) {
                size_t wi = weight_out_in ? size_t(c) * in_dim + k : size_t(k) * out_dim + c;
                acc = f_add(acc, f_mul(load_typed(x, size_t(r) * in_dim + k, dtype), load_typed(w, wi, dtype)));
            }
            store_typed(out, size_t(r) * out_dim + c, dtype, acc);
        }
    }
}

// vyre-libs/src/math/linalg/matmul.rs:17-60 and nn/linear/inner/builder.rs:363-391:
// out[m,n] = sum_k a[m,k]*b[k,n] (+bias[n]) in wrapping u32.
VYO_API void vyo_matmul_u32(const uint32_t* a, const uint32_t* b, const uint32_t* bias, uint32_t* out,
                            uint32_t m, uint32_t k, uint32_t n) {
#pragma omp parallel for schedule(static)
    for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < n; ++j) {
            uint32_t acc = 0;
            for (uint32_t kk = 0; kk < k; ++kk) acc += a[size_t(i) * k + kk] * b[size_t(kk) * n + j];
            if (bias) acc += bias[j];
            out[size_t(i) * n + j] = acc;
        }
}

// ---------------------------------------------------------------------------------------------
// MoE gating - vyre-libs/src/nn/moe/gating.rs:71-147 + vyre-primitives/src/nn/quest_paging_passes.rs:169-202
// max (init f32::MIN), sum exp(s-max) in index order, k rounds of strict-'>' argmax with the winner
// overwritten by the f32::MIN sentinel, weight = exp(s_best - max) / sum (softmax over ALL experts).
// ---------------------------------------------------------------------------------------------
VYO_API void vyo_moe_gate(const float* scores, uint32_t num_experts, uint32_t k, uint32_t* out_idx,
                          float* out_w) {
    const float fmin = std::numeric_limits<float>::lowest();
    std::vector<float> scratch(num_experts);
    float mx = fmin;
    for (uint32_t i = 0; i < num_experts; ++i) {
        scratch[i] = canon(scores[i]);
        mx = f_max(mx, scores[i]);
    }
    float sum = 0.0f;
    for (uint32_t i = 0; i < num_experts; ++i) sum = f_add(sum, f_exp(f_sub(scores[i], mx)));
    for (uint32_t j = 0; j < k; ++j) {
        uint32_t best = 0;
        float bs = fmin;
        for (uint32_t q = 0; q < num_experts; ++q) {
            if (scratch[q] > bs) { bs = scratch[q]; best = q; }
        }
        out_idx[j] = best;
        scratch[best] = fmin;
    }
    for (uint32_t j = 0; j < k; ++j) out_w[j] = f_div(f_exp(f_sub(scores[out_idx[j]], mx)), sum);
}

// vyre-libs/src/nn/moe/topk_selection.rs:6-135: k slots sorted descending, insertion on strict '>'
// (ties keep the earlier index), slots init (-inf, 0).
static void topk_insert(std::vector<float>& vals, std::vector<uint32_t>& idxs, uint32_t k, float v, uint32_t i) {
    uint32_t pos = k;
    for (uint32_t j = 0; j < k; ++j)
        if (pos == k && v > vals[j]) pos = j;
    if (pos < k) {
        for (uint32_t rev = k - 1; rev > pos; --rev) { vals[rev] = vals[rev - 1]; idxs[rev] = idxs[rev - 1]; }
        vals[pos] = v;
        idxs[pos] = i;
    }
}
// vyre-libs/src/nn/moe/softmax_top_k.rs:25-101: returns [out_indices, out_weights, best_vals, best_idxs].
VYO_API void vyo_softmax_top_k(const float* scores, uint32_t n, uint32_t k, uint32_t* out_idx, float* out_w,
                               float* best_vals, uint32_t* best_idxs) {
    std::vector<float> vals(k, -std::numeric_limits<float>::infinity());
    std::vector<uint32_t> idxs(k, 0);
    float mx = -std::numeric_limits<float>::infinity();
    for (uint32_t i = 0; i < n; ++i)
        if (canon(scores[i]) > mx) mx = canon(scores[i]);
    float sum = 0.0f;
    for (uint32_t i = 0; i < n; ++i) {
        float e = f_exp(f_sub(scores[i], mx));
        sum = f_add(sum, e);
        topk_insert(vals, idxs, k, e, i);
    }
    for (uint32_t s = 0; s < k; ++s) {
        out_w[s] = f_div(vals[s], sum);
        out_idx[s] = idxs[s];
        best_vals[s] = vals[s];
        best_idxs[s] = idxs[s];
    }
}
// vyre-libs/src/nn/moe/top_k.rs:18-60
VYO_API void vyo_top_k(const float* input, uint32_t n, uint32_t k, uint32_t* out_idx) {
    std::vector<float> vals(k, -std::numeric_limits<float>::infinity());
    std::vector<uint32_t> idxs(k, 0);
    for (uint32_t i = 0; i < n; ++i) topk_insert(vals, idxs, k, canon(input[i]), i);
    for (uint32_t s = 0; s < k; ++s) out_idx[s] = idxs[s];
}

// vyre-libs/src/nn/activation/unary.rs:79-100 + swiglu.rs:17-48:
// out = cast(dtype, gate * (up * (1/(1+exp(-gate))))) with f32 math.
static inline float swiglu_f32(float g, float u) {
    float sig = f_div(1.0f, f_add(1.0f, f_exp(f_neg(g))));
    return f_mul(g, f_mul(u, sig));
}
VYO_API void vyo_swiglu(const void* gate, const void* up, void* out, uint32_t n, uint32_t dtype) {
    for (uint32_t i = 0; i < n; ++i)
        store_typed(out, i, dtype, swiglu_f32(load_typed(gate, i, dtype), load_typed(up, i, dtype)));
}

// vyre-libs/src/nn/moe/expert_mlp.rs:18-150: f32, weights [in,hidden] / [hidden,out];
// hidden_h = (g*sigmoid(g))*u; out[o] = b_d[o] + sum_h hidden_h*w_d[h,o]; all sequential mul-then-add.
VYO_API void vyo_expert_mlp(const float* x, const float* wg, const float* bg, const float* wu, const float* bu,
                            const float* wd, const float* bd, float* out, uint32_t in_dim, uint32_t hidden,
                            uint32_t out_dim) {
    std::vector<float> hid(hidden);
#pragma omp parallel for schedule(static)
    for (uint32_t h = 0; h < hidden; ++h) {
        float g = canon(bg[h]), u = canon(bu[h]);
        for (uint32_t k = 0; k < in_dim; ++k) {
            g = f_add(g, f_mul(x[k], wg[size_t(k) * hidden + h]));
            u = f_add(u, f_mul(x[k], wu[size_t(k) * hidden + h]));
        }
        float sig = f_div(1.0f, f_add(1.0f, f_exp(f_neg(g))));
        hid[h] = f_mul(f_mul(g, sig), u);
    }
#pragma omp parallel for schedule(static)
    for (uint32_t o = 0; o < out_dim; ++o) {
        float acc = canon(bd[o]);
        for (uint32_t h = 0; h < hidden; ++h) acc = f_add(acc, f_mul(hid[h], wd[size_t(h) * out_dim + o]));
        out[o] = acc;
    }
}

// vyre-libs/src/nn/moe/moe_layer.rs:57-101: out[j] = sum_{e<k} w[e]*expert_out[e,j], sequential e.
VYO_API void vyo_moe_layer_accumulate(const float* weights, const float* expert_out, float* out, uint32_t k,
                                      uint32_t out_dim) {
    for (uint32_t j = 0; j < out_dim; ++j) {
        float acc = 0.0f;
        for (uint32_t e = 0; e < k; ++e) acc = f_add(acc, f_mul(weights[e], expert_out[size_t(e) * out_dim + j]));
        out[j] = acc;
    }
}

// ---------------------------------------------------------------------------------------------
// Compositions for the benchmark configurations. These dtype mixes are NOT pinned by any reference
// fixture (the reference op is f32 with f32 scales and u32 zero points); they compose the pinned
// pieces above: bf16 conversion (float16.rs), the row-major signed-int4 primitive layout
// (cpu.rs:35-61, programs.rs:181) read as offset-binary with zero point 8, f32 FMA semantics.
// ---------------------------------------------------------------------------------------------

// Row-major K-inner int4 linear with per-group scales:
//   W packed u4 [N, K/2 bytes] (byte j of a row holds k=2j in the low nibble, k=2j+1 in the high
//   nibble, i.e. the primitive u32 word layout), value q in 0..15, zero point `zp_const`;
//   scale bf16 [N, K/group]; x bf16 [M, K]; out dtype bf16 or f32, [M, N].
// mode 0: exact products accumulated in f64, one rounding to f32, then the output cast
//         ("f32 accumulate" contract, order-independent reference value).
// mode 1: weights first dequantised to bf16 = rne((q-zp)*s) as the prefill tensor-core path stores
//         them, then accumulated in f64.
VYO_API void vyo_int4_rowmajor_linear(const uint16_t* x_bf16, const uint8_t* w_packed, const uint16_t* scale_bf16,
                                      void* out, uint32_t m, uint32_t n, uint32_t k, uint32_t group,
                                      int32_t zp_const, uint32_t out_dtype, uint32_t mode) {
    const uint32_t groups = (k + group - 1) / group;
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < n; ++r) {
        const uint8_t* wr = w_packed + size_t(r) * (k / 2);
        std::vector<double> wq(k);
        for (uint32_t kk = 0; kk < k; ++kk) {
            uint8_t byte = wr[kk / 2];
            int32_t q = (kk & 1) ? (byte >> 4) : (byte & 0xF);
            float s = bf16_to_f32(scale_bf16[size_t(r) * groups + kk / group]);
            float prod = f_mul(float(q - zp_const), s);  // exact: 5-bit x 8-bit significands
            wq[kk] = (mode == 1) ? double(bf16_to_f32(f32_to_bf16(prod))) : double(prod);
        }
        for (uint32_t b = 0; b < m; ++b) {
            const uint16_t* xb = x_bf16 + size_t(b) * k;
            double acc = 0.0;
            for (uint32_t kk = 0; kk < k; ++kk) acc += double(bf16_to_f32(xb[kk])) * wq[kk];
            store_typed(out, size_t(b) * n + r, out_dtype, float(acc));
        }
    }
}

// int8 weight-only linear (benchmark config 1): Y[m,n] = sum_k X[m,k]*(f32(W[n,k])*s[n]),
// W int8 [N,K] signed, per-output-channel f32 scale; composition of int8_unpack (f32(value)*scale[row],
// int8.rs:15-50, here with a signed value) and linear_rows_no_bias_out_in (builder.rs:241, f32 sequential).
// mode 0: f64 accumulation of exact products then one rounding; mode 1: reference f32 sequential order.
VYO_API void vyo_int8_weight_only_linear(const float* x, const int8_t* w, const float* scale, float* out,
                                         uint32_t m, uint32_t n, uint32_t k, uint32_t mode) {
#pragma omp parallel for collapse(2) schedule(static)
    for (uint32_t r = 0; r < m; ++r) {
        for (uint32_t c = 0; c < n; ++c) {
            const int8_t* wr = w + size_t(c) * k;
            const float* xr = x + size_t(r) * k;
            if (mode == 1) {
                float acc = 0.0f;
                for (uint32_t kk = 0; kk < k; ++kk) acc = f_add(acc, f_mul(xr[kk], f_mul(float(wr[kk]), scale[c])));
                out[size_t(r) * n + c] = acc;
            } else {
                double acc = 0.0;
                for (uint32_t kk = 0; kk < k; ++kk) acc += double(xr[kk]) * double(f_mul(float(wr[kk]), scale[c]));
                out[size_t(r) * n + c] = canon(float(acc));
            }
        }
    }
}

// Per-token symmetric int8 quantisation (unpinned in the reference; rule fixed here):
//   s_t = max_k |x_tk| / 127 (f32), q = clamp(rne(x / s_t), -127, 127); an all-zero row gets s_t = 1 and q = 0.
VYO_API void vyo_quantize_per_token_int8(const uint16_t* x_bf16, int8_t* q, float* scales, uint32_t m, uint32_t k) {
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < m; ++r) {
        float amax = 0.0f;
        for (uint32_t kk = 0; kk < k; ++kk) amax = std::fmax(amax, std::fabs(bf16_to_f32(x_bf16[size_t(r) * k + kk])));
        float s = amax > 0.0f ? amax / 127.0f : 1.0f;
        scales[r] = s;
        for (uint32_t kk = 0; kk < k; ++kk) {
            float v = bf16_to_f32(x_bf16[size_t(r) * k + kk]) / s;
            float rn = std::nearbyintf(v);  // round-to-nearest-even under the default rounding mode
            rn = std::fmin(127.0f, std::fmax(-127.0f, rn));
            q[size_t(r) * k + kk] = int8_t(rn);
        }
    }
}

// int8 x int8 -> int32 GEMM, out[m,n] = sum_k a[m,k]*w[n,k] with wrapping 32-bit arithmetic - the
// two's-complement reading of the reference's wrapping-u32 matmul (matmul.rs:17-60) on sign-extended int8.
// rows [row_begin,row_end) only, so a sampled slice of a large problem can be checked/timed.
VYO_API void vyo_int8_gemm_i32(const int8_t* a, const int8_t* w, int32_t* out, uint32_t m, uint32_t n, uint32_t k,
                               uint32_t row_begin, uint32_t row_end) {
    (void)m;
#pragma omp parallel for schedule(static)
    for (uint32_t c = 0; c < n; ++c) {
        const int8_t* wr = w + size_t(c) * k;
        for (uint32_t r = row_begin; r < row_end; ++r) {
            const int8_t* ar = a + size_t(r) * k;
            uint32_t acc = 0;
            for (uint32_t kk = 0; kk < k; ++kk) acc += uint32_t(int32_t(ar[kk])) * uint32_t(int32_t(wr[kk]));
            out[size_t(r - row_begin) * n + c] = int32_t(acc);
        }
    }
}

// MoE FFN layer for a list of tokens (benchmark config 4), composed per token from the single-token
// reference ops: router logits = linear_rows_no_bias_out_in_typed(bf16) (builder.rs:241), moe_gate
// (gating.rs:19-69) on the f32 view of the bf16 logits, per selected expert
// h = swiglu_typed(bf16)(w1 x, w3 x) (swiglu.rs:26), y_e = w2 h (int4 row-major linears above, bf16
// out), out = cast_bf16(sum_e weight_e * y_e) in selection order (moe_layer.rs:57-101).
// tokens: indices into x of the tokens to evaluate (so a sample of a large batch can be checked).
// Expert weights are stacked: w13 = [E][2][H][K/2] (w1 then w3), s13 = [E][2][H][K/G]; w2 = [E][K][H/2], s2 = [E][K][H/G].
// Also returns the routing (top-k indices and weights) for each evaluated token.
// weight_mode: 0 = dequantised weights exact (the decode kernels' arithmetic), 1 = each dequantised weight rounded to
// bf16 first (what a tensor-core path that materialises bf16 weight tiles computes); see vyo_int4_rowmajor_linear.
VYO_API void vyo_moe_ffn_int4(const uint16_t* x_bf16, const uint16_t* w_router_bf16, const uint8_t* w13,
                              const uint16_t* s13, const uint8_t* w2, const uint16_t* s2, const uint32_t* tokens,
                              uint32_t n_tokens, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t topk,
                              uint32_t group, uint32_t weight_mode, uint16_t* out_bf16, uint32_t* out_idx, float* out_w) {
    const size_t w1_bytes = size_t(inter) * (hidden / 2);
    const size_t s1_elems = size_t(inter) * (hidden / group);
    const size_t w2_bytes = size_t(hidden) * (inter / 2);
    const size_t s2_elems = size_t(hidden) * (inter / group);
    for (uint32_t t = 0; t < n_tokens; ++t) {
        const uint16_t* xt = x_bf16 + size_t(tokens[t]) * hidden;
        std::vector<uint16_t> logits_bf16(experts);
        vyo_linear_rows(xt, w_router_bf16, nullptr, logits_bf16.data(), 1, hidden, experts, DT_BF16, 1);
        std::vector<float> logits(experts);
        for (uint32_t e = 0; e < experts; ++e) logits[e] = bf16_to_f32(logits_bf16[e]);
        std::vector<uint32_t> idx(topk);
        std::vector<float> wts(topk);
        vyo_moe_gate(logits.data(), experts, topk, idx.data(), wts.data());
        std::vector<float> acc(hidden, 0.0f);
        std::vector<uint16_t> g(inter), u(inter), h(inter), y(hidden);
        for (uint32_t j = 0; j < topk; ++j) {
            uint32_t e = idx[j];
            const uint8_t* w1 = w13 + size_t(e) * 2 * w1_bytes;
            const uint8_t* w3 = w1 + w1_bytes;
            const uint16_t* s1 = s13 + size_t(e) * 2 * s1_elems;
            const uint16_t* s3 = s1 + s1_elems;
            vyo_int4_rowmajor_linear(xt, w1, s1, g.data(), 1, inter, hidden, group, 8, DT_BF16, weight_mode);
            vyo_int4_rowmajor_linear(xt, w3, s3, u.data(), 1, inter, hidden, group, 8, DT_BF16, weight_mode);
            vyo_swiglu(g.data(), u.data(), h.data(), inter, DT_BF16);
            vyo_int4_rowmajor_linear(h.data(), w2 + size_t(e) * w2_bytes, s2 + size_t(e) * s2_elems, y.data(), 1,
                                     hidden, inter, group, 8, DT_BF16, weight_mode);
            for (uint32_t c = 0; c < hidden; ++c) acc[c] = f_add(acc[c], f_mul(wts[j], bf16_to_f32(y[c])));
            out_idx[size_t(t) * topk + j] = e;
            out_w[size_t(t) * topk + j] = wts[j];
        }
        for (uint32_t c = 0; c < hidden; ++c) out_bf16[size_t(t) * hidden + c] = f32_to_bf16(acc[c]);
    }
}

VYO_API int vyo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ---- the operators either side of the feed-forward block, and the GGML K-quant linears ---------------------------

// vyre-libs/src/nn/activation/residual_add.rs:10-52 over unary.rs:44-76: out = cast(dtype, f32(residual) + f32(branch))
VYO_API void vyo_residual_add(const void* residual, const void* branch, void* out, uint32_t n, uint32_t dtype) {
    for (uint32_t i = 0; i < n; ++i) store_typed(out, i, dtype, f_add(load_typed(residual, i, dtype), load_typed(branch, i, dtype)));
}

// vyre-libs/src/nn/norm/gated_rms_norm.rs:123-247. Per element: sum_squares = sequential f32 sum of x^2 over the row;
// normalized = x * (1 / sqrt(sum_squares / hidden + eps))  (InverseSqrt = 1.0 / sqrtf, vyre-reference/src/ieee754.rs:60-70);
// rounded to dtype; times f32(weight[col]); with a gate: times gate / (1 + exp(-gate)); one final cast to dtype.
// Pinned by the known answers of vyre-libs/tests/gated_rms_norm_contract.rs (f32 fixture, exact F16 / BF16 words, F32 scales).
VYO_API void vyo_rms_norm(const void* input, const void* weight, const void* gate, void* out, uint32_t rows, uint32_t hidden,
                          float eps, uint32_t dtype, uint32_t weight_dtype) {
    for (uint32_t r = 0; r < rows; ++r) {
        float sum = 0.0f;
        for (uint32_t c = 0; c < hidden; ++c) {
            const float v = load_typed(input, size_t(r) * hidden + c, dtype);
            sum = f_add(sum, f_mul(v, v));
        }
        const float inv = f_div(1.0f, canon(std::sqrt(canon(f_add(f_div(sum, float(hidden)), eps)))));
        for (uint32_t c = 0; c < hidden; ++c) {
            const size_t i = size_t(r) * hidden + c;
            float normalized = f_mul(load_typed(input, i, dtype), inv);
            if (dtype == DT_BF16) normalized = bf16_to_f32(f32_to_bf16(normalized));
            else if (dtype == DT_F16) normalized = f16_to_f32(f32_to_f16(normalized));
            float v = f_mul(normalized, load_typed(weight, c, weight_dtype));
            if (gate) {
                const float g = load_typed(gate, i, dtype);
                v = f_mul(v, f_div(g, f_add(1.0f, f_exp(f_neg(g)))));
            }
            store_typed(out, i, dtype, v);
        }
    }
}

// vyre-libs/src/nn/quant/ggml.rs:28-120 (k_quant_unpack): bits = 4 (Q4_K: blocks of 32, 4 words) or 2 (Q2_K: blocks
// of 16, 1 word); out[i] = f32(q_i) * scale[block] + min[block]
static inline uint32_t k_quant_value(const uint32_t* packed, uint32_t linear, uint32_t bits, uint32_t* block) {
    const uint32_t block_size = bits == 4 ? 32u : 16u, values_per_byte = 8u / bits, words_per_block = bits == 4 ? 4u : 1u;
    const uint32_t block_idx = linear / block_size, within = linear % block_size;
    const uint32_t byte_idx = within / values_per_byte, value_shift = (within % values_per_byte) * bits;
    const uint32_t word = packed[size_t(block_idx) * words_per_block + byte_idx / 4];
    *block = block_idx;
    return (word >> ((byte_idx % 4) * 8 + value_shift)) & ((1u << bits) - 1u);
}
VYO_API void vyo_k_quant_unpack(const uint32_t* packed, const float* scales, const float* mins, float* out, uint32_t n,
                                uint32_t bits) {
    for (uint32_t i = 0; i < n; ++i) {
        uint32_t block;
        const uint32_t q = k_quant_value(packed, i, bits, &block);
        out[i] = f_add(f_mul(float(q), scales[block]), mins[block]);
    }
}
// ggml.rs:217-333 (k_quant_linear): out[i] = b[i] + sum_k x[k] * (q(k * out_dim + i) * scale + min), k ascending,
// every product and sum rounded on its own
VYO_API void vyo_k_quant_linear(const float* x, const uint32_t* packed, const float* scales, const float* mins, const float* b,
                                float* out, uint32_t in_dim, uint32_t out_dim, uint32_t bits) {
    for (uint32_t i = 0; i < out_dim; ++i) {
        float acc = canon(b[i]);
        for (uint32_t k = 0; k < in_dim; ++k) {
            uint32_t block;
            const uint32_t q = k_quant_value(packed, k * out_dim + i, bits, &block);
            const float weight = f_add(f_mul(float(q), scales[block]), mins[block]);
            acc = f_add(acc, f_mul(x[k], weight));
        }
        out[i] = acc;
    }
}
