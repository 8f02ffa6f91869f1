// Timed CPU baseline of the decode GEMV (test / bench infrastructure, never linked into the product library).
//
// This is the reference bench's own CPU loop (vyre-bench/src/cases/quantized_linear.rs:447-463: one task per output,
// sequential k, `acc += x[k] * ((nibble - zero_point) * scale)` in f32, tasks spread over the host cores as rayon's
// into_par_iter does) restated for the row-major layout of the benchmark's second configuration: packed bytes
// [n, k/2] (element 2j in the low nibble), bf16 scale per 128-k group, constant zero point 8, f32 activations.
// It is NOT the checker (that is the f64-accumulating oracle); it exists to be timed beside the GPU number, built
// with -O3 for a fair figure.
#include <stdint.h>
#include <string.h>

#include <cstddef>

extern "C" void vyo_cpu_baseline_int4_gemv(const float* x, const uint8_t* w_packed, const uint16_t* scale_bf16, float* out,
                                           uint32_t m, uint32_t n, uint32_t k, uint32_t group, int32_t zero_point) {
    const uint32_t groups = k / group;
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < n; ++r) {
        const uint8_t* wr = w_packed + size_t(r) * (k / 2);
        for (uint32_t b = 0; b < m; ++b) {
            const float* xb = x + size_t(b) * k;
            float acc = 0.0f;
            for (uint32_t g = 0; g < groups; ++g) {
                const uint32_t bits = uint32_t(scale_bf16[size_t(r) * groups + g]) << 16;
                float s;
                memcpy(&s, &bits, 4);
                for (uint32_t kk = g * group; kk < (g + 1) * group; kk += 2) {
                    const uint8_t byte = wr[kk / 2];
                    acc += xb[kk] * (float(int32_t(byte & 0xF) - zero_point) * s);
                    acc += xb[kk + 1] * (float(int32_t(byte >> 4) - zero_point) * s);
                }
            }
            out[size_t(b) * n + r] = acc;
        }
    }
}
