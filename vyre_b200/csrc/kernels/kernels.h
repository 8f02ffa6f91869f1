// Launch prototypes of the hand-written sm_100a kernels. All pointers are device pointers; every launcher
// returns the cudaError_t of the launch (0 = ok) and never synchronises.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace vybk {

struct PeerGather;  // defined below: the peer addresses of a gather

// ---- decode GEMV / skinny GEMM (int4_gemv.cu) ---------------------------------------------------------------
// y[m,n] = cast( sum_k x[m,k] * (q[n,k]-8) * s[n,k/128] ), m <= 8, group 128, k % 1024 == 0.
// out_dtype: 0 = bf16, 1 = f32. status: optional 4-word device buffer set non-zero when a bounded wait ran out.
bool int4_gemv_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group);
cudaError_t launch_int4_gemv(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                             uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                             uint32_t* status, bool constant_weights = false);
// half-SM form (int4_gemv_halfsm.cu): m <= 4, k 2048 or 4096; launch_int4_gemv routes to it
// rows longer than 4096 (k a multiple of 2048), m <= 4: one launch of the k-block form per 4096 / 2048 columns, sums carried in f32
bool int4_gemv_kblocks_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group);
// resid / gate (bf16 [m][n], bf16 outputs only, at most one): the residual add or SwiGLU(gate, this projection) applied to the
// rounded sums in the launch when it runs as ONE launch (*stores_fused = true); the launch-per-block fallback leaves the
// plain projection in y (*stores_fused = false)
cudaError_t launch_int4_gemv_kblocks(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                     uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                                     bool constant_weights, const void* resid = nullptr, const void* gate = nullptr,
                                     bool* stores_fused = nullptr);
// f16 tensor path of the same launch shape (int4_gemv_batch8.cu): up to eight batch rows in one launch, k 2048 or 4096
bool int4_gemv_batch8_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group);
cudaError_t launch_int4_gemv_batch8(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                    uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                                    bool constant_weights);
bool int4_gemv_halfsm_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group);
cudaError_t launch_int4_gemv_halfsm(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                    uint32_t n, uint32_t k, uint32_t out_f32, int sm_count, cudaStream_t stream,
                                    uint32_t* status, bool constant_weights, const PeerGather* gather = nullptr,
                                    uint32_t half = 0, bool pipelined = false,
                                    // the residual block around the projection, m <= 2, bf16 outputs: learned RMSNorm of x
                                    // (bf16 weight [k]) in the prologue, residual (bf16 [m][n]) added in the output stores
                                    // or, instead of the residual, SwiGLU(gate, this projection) with gate bf16 [m][n]
                                    const void* norm_w = nullptr, float norm_eps = 0.0f, const void* resid = nullptr,
                                    const void* gate = nullptr);
// ---- all-gather of column-parallel outputs over peer memory (allgather_push.cu) ------------------------------------
// gather buffers [2][world][m][n] bf16 per rank; arrival counters and launch counters are 32-bit device words,
// zero before the first push
struct PeerGather {
    uint32_t world = 0, rank = 0;
    unsigned long long peer_out[8] = {};   // base of every rank's gather buffer (own rank included)
    unsigned long long peer_flag[8] = {};  // every rank's 256 bytes of arrival counters: word 8 s counts pushes from rank s
    unsigned long long epoch = 0;          // local: 8 words, pushes completed per peer slot
    unsigned long long wait_clocks = 0;    // clock limit of a device-side wait; 0 = about 2 s
    unsigned long long slots = 0;          // slots of the gather buffer ([slots][world][m][n]); 0 = two halves
};
cudaError_t launch_allgather_push(const PeerGather& ag, uint32_t half, uint32_t m, uint32_t n, cudaStream_t stream,
                                  uint32_t* status);
cudaError_t launch_allgather_wait(const PeerGather& ag, cudaStream_t stream, uint32_t* status);
// column-parallel gather: this rank's [rows, row_bytes] block -> byte offset dst_offset_bytes (row pitch dst_pitch_bytes)
// of EVERY rank's buffer peer_out[r], own rank included; tickets: 8 zeroed local words; then every destination's
// counter for this rank goes up by one. launch_colpar_wait: until every rank has delivered `want` blocks here.
cudaError_t launch_colpar_push(const PeerGather& ag, const void* src, uint32_t rows, uint32_t row_bytes, uint64_t dst_pitch_bytes,
                               uint64_t dst_offset_bytes, uint32_t* tickets, cudaStream_t stream, uint32_t* status);
cudaError_t launch_colpar_wait(const PeerGather& ag, uint32_t want, cudaStream_t stream, uint32_t* status);
// any group size dividing k, k % 8 == 0, any m; plain loads, no TMA
cudaError_t launch_int4_linear_generic(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y,
                                       uint32_t m, uint32_t n, uint32_t k, uint32_t group, uint32_t out_f32,
                                       cudaStream_t stream);

// ---- int8 weight-only linear (int8_linear.cu) ------------------------------------------------------------------
cudaError_t launch_int8_weight_only_linear(const float* x, const int8_t* w, const float* scale, float* y, uint32_t m,
                                           uint32_t n, uint32_t k, cudaStream_t stream);

// ---- int4 prefill GEMM on tcgen05 with in-kernel dequantisation (int4_prefill_tcgen05.cu) -------------------------
bool int4_prefill_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group);
cudaError_t launch_int4_prefill(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                uint32_t n, uint32_t k, uint32_t group, uint32_t out_f32, int sm_count,
                                cudaStream_t stream, uint32_t* status);

// ---- int4 GEMM on CTA pairs (int4_gemm_pair_tcgen05.cu): dense, grouped per expert, grouped + SwiGLU ---------------
// plain: y[m, n] over weights [experts][n][k/2]; glu: h[m, n] = swiglu over weights [experts][2][n][k/2] (W1 then W3).
// tile_expert / m_tiles_dev (device pointers, optional) describe 256-row tiles of an expert-sorted, 256-padded
// activation buffer; without them every row uses expert 0.
bool int4_gemm_pair_supported(uint32_t m, uint32_t n, uint32_t k, uint32_t group);
cudaError_t launch_int4_gemm_pair(const void* x_bf16, const void* w_packed, const void* scale_bf16, void* y, uint32_t m,
                                  uint32_t n, uint32_t k, uint32_t group, uint32_t out_f32, uint32_t glu, uint32_t experts,
                                  const uint32_t* tile_expert, const uint32_t* m_tiles_dev, uint32_t ldy, int sm_count,
                                  cudaStream_t stream, uint32_t* status);

// ---- multi-token int4 MoE FFN layer (moe_ffn.cu): router + gate, permutation, grouped GEMMs, combine -------------
bool moe_ffn_int4_supported(uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t topk,
                            uint32_t group);
size_t moe_ffn_int4_scratch_bytes(uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t topk);
cudaError_t launch_moe_ffn_int4(const void* x_bf16, const void* w_router_bf16, const void* w13, const void* s13,
                                const void* w2, const void* s2, void* out_bf16, uint32_t* routing_idx, float* routing_w,
                                void* scratch, uint32_t tokens, uint32_t hidden, uint32_t inter, uint32_t experts,
                                uint32_t topk, uint32_t group, int sm_count, cudaStream_t stream, uint32_t* status);

// the stages of the layer on their own (expert-parallel runs put an exchange between them)
cudaError_t launch_moe_route(const void* x_bf16, const void* w_router_bf16, uint32_t* routing_idx, float* routing_w,
                             uint32_t tokens, uint32_t hidden, uint32_t experts, uint32_t topk, cudaStream_t stream);
cudaError_t launch_rows_gather_bf16(const void* src, const uint32_t* index, void* dst, uint32_t rows, uint32_t row_elems,
                                    int sm_count, cudaStream_t stream);
cudaError_t launch_moe_experts_int4(const void* x_sorted, const void* w13, const void* s13, const void* w2, const void* s2,
                                    void* y_rows, void* h_scratch, const uint32_t* tile_expert, const uint32_t* m_tiles_dev,
                                    uint32_t max_rows, uint32_t hidden, uint32_t inter, uint32_t experts, uint32_t group,
                                    int sm_count, cudaStream_t stream, uint32_t* status);
cudaError_t launch_moe_combine(const void* y_rows, const uint32_t* pos, const float* routing_w, void* out_bf16,
                               uint32_t tokens, uint32_t hidden, uint32_t topk, int sm_count, cudaStream_t stream);

// ---- expert-parallel MoE FFN with device-side dispatch / combine over peer memory (moe_ep.cu) -----------------------
struct MoeEp {
    uint32_t world = 0, rank = 0;
    unsigned long long peer_base[8] = {};  // base of every rank's symmetric region (own rank included)
    unsigned long long off_counts = 0, off_flags = 0, off_src = 0, off_xg = 0, off_yhome = 0;  // same on every rank
    unsigned long long wait_clocks = 0;  // clock limit of a device-side wait; 0 = about 2 s
};
uint32_t moe_ep_max_rows(uint32_t tokens_total, uint32_t experts, uint32_t topk, uint32_t world);
void moe_ep_symmetric_layout(uint32_t tokens_local_max, uint32_t tokens_total, uint32_t hidden, uint32_t experts,
                             uint32_t topk, uint32_t world, MoeEp* c, size_t* total_bytes);
size_t moe_ep_local_bytes(uint32_t tokens_local_max, uint32_t tokens_total, uint32_t hidden, uint32_t inter, uint32_t experts,
                          uint32_t topk, uint32_t world);
cudaError_t launch_moe_ep_ffn(const MoeEp& c, const void* x_bf16, const void* w_router_bf16, const void* w13, const void* s13,
                              const void* w2, const void* s2, void* out_bf16, uint32_t* routing_idx, float* routing_w,
                              void* local_scratch, uint32_t tokens, uint32_t tokens_total, uint32_t hidden, uint32_t inter,
                              uint32_t experts, uint32_t topk, uint32_t group, int sm_count, cudaStream_t stream,
                              uint32_t* status);

// ---- int8 x int8 -> int32 GEMM on tcgen05 + per-token activation quantiser (int8_gemm_tcgen05.cu) --------------
bool int8_gemm_supported(uint32_t m, uint32_t n, uint32_t k);
cudaError_t launch_int8_gemm(const int8_t* a, const int8_t* w, int32_t* out, uint32_t m, uint32_t n, uint32_t k,
                             int sm_count, cudaStream_t stream, uint32_t* status);
// CTA-pair form (int8_gemm_pair_tcgen05.cu): 256 x 256 tiles on two SMs; launch_int8_gemm uses it from two waves of pair tiles on
bool int8_gemm_pair_supported(uint32_t m, uint32_t n, uint32_t k);
// Where a gathering GEMM stores its int32 outputs: the same [m, n] block at element offset col_off (row pitch `pitch`
// elements) of `count` buffers, normally every rank's full output (peer addresses). count == 0: the plain `out`.
struct GemmGatherOut {
    unsigned long long dst[8] = {};
    uint32_t count = 0, pad = 0;
    unsigned long long pitch = 0, col_off = 0;
};
cudaError_t launch_int8_gemm_pair_gather(const int8_t* a, const int8_t* w, const GemmGatherOut& go, uint32_t m, uint32_t n,
                                         uint32_t k, int sm_count, cudaStream_t stream, uint32_t* status);
cudaError_t launch_colpar_signal(const PeerGather& ag, cudaStream_t stream);
cudaError_t launch_int8_gemm_pair(const int8_t* a, const int8_t* w, int32_t* out, uint32_t m, uint32_t n, uint32_t k,
                                  int sm_count, cudaStream_t stream, uint32_t* status);
cudaError_t launch_quantize_per_token_int8(const void* x_bf16, int8_t* q, float* scales, uint32_t m, uint32_t k,
                                           cudaStream_t stream);

// ---- tensor-core peak microbenchmark (tensor_peak.cu): MMAs from shared-memory operands only; for the bench's roofline
cudaError_t launch_tensor_peak(uint32_t int8, uint32_t iters, int sm_count, cudaStream_t stream, uint32_t* status,
                               double* ops_per_launch);

// ---- the same two kernels with the quantised activations in a fixed device array (int8_dynamic_static_scratch.cu)
size_t int8_dynamic_static_scratch_limit();
cudaError_t launch_int8_dynamic_static_scratch(const void* x_bf16, const int8_t* w, float* x_scale, int32_t* y,
                                               uint32_t m, uint32_t n, uint32_t k, int sm_count, cudaStream_t stream,
                                               uint32_t* status);

// ---- reference-shaped small ops (ref_ops.cu); each keeps the reference's evaluation order -----------------------
cudaError_t launch_linear_4bit(const float* x, const uint32_t* w, const float* b, float* out, uint32_t in_dim,
                               uint32_t out_dim, cudaStream_t s);
cudaError_t launch_linear_4bit_affine_grouped(const float* x, const uint32_t* w, const float* scale,
                                              const uint32_t* zp, const float* b, float* out, uint32_t in_dim,
                                              uint32_t out_dim, uint32_t group, uint32_t batch, cudaStream_t s);
cudaError_t launch_i4_unpack(const uint32_t* packed, int32_t* out, uint32_t lanes, cudaStream_t s);
cudaError_t launch_i4_dot_i32(const uint32_t* lhs, const uint32_t* rhs, int32_t* out, uint32_t lanes, cudaStream_t s);
cudaError_t launch_i4_dot_f32_scaled(const uint32_t* lhs, const uint32_t* rhs, const float* ls, const float* rs,
                                     float* out, uint32_t lanes, cudaStream_t s);
cudaError_t launch_i4_batched_matvec(const uint32_t* w, const float* x, const float* scales, float* out,
                                     uint32_t batch, uint32_t rows, uint32_t cols, cudaStream_t s);
cudaError_t launch_i4_batched_matmul(const uint32_t* w, const uint32_t* act, const float* rs, const float* bs,
                                     float* out, uint32_t batch, uint32_t rows, uint32_t cols, cudaStream_t s);
cudaError_t launch_i4_batched_matmul_top1(const uint32_t* w, const uint32_t* act, const float* rs, const float* bs,
                                          float* out, uint32_t batch, uint32_t rows, uint32_t cols, cudaStream_t s);
cudaError_t launch_int8_unpack(const uint32_t* packed, const float* scales, float* out, uint32_t n, uint32_t cols,
                               cudaStream_t s);
cudaError_t launch_int8_pack(const uint32_t* in, uint32_t* out, uint32_t n, cudaStream_t s);
// ---- the same two reference operators at large shapes (dropin_fast.cu): the reference's layouts and dequantisation,
// a summation order of their own. The *_supported predicates are pure functions of the op spec.
bool affine_grouped_fast_supported(uint32_t in_dim, uint32_t out_dim, uint32_t group, uint32_t batch);
bool i4_matvec_fast_supported(uint32_t batch, uint32_t rows, uint32_t cols);
cudaError_t launch_affine_grouped_fast(const float* x, const uint32_t* w, const float* scale, const uint32_t* zp,
                                       const float* b, float* out, uint32_t in_dim, uint32_t out_dim, uint32_t group,
                                       uint32_t batch, int sm_count, cudaStream_t s);
cudaError_t launch_i4_matvec_fast(const uint32_t* w, const float* x, const float* scales, float* out, uint32_t batch,
                                  uint32_t rows, uint32_t cols, cudaStream_t s);
// dtype: 0 = f32, 1 = bf16, 2 = f16
cudaError_t launch_linear_rows(const void* x, const void* w, const void* bias, void* out, uint32_t rows,
                               uint32_t in_dim, uint32_t out_dim, uint32_t dtype, uint32_t out_in, cudaStream_t s);
cudaError_t launch_matmul_u32(const uint32_t* a, const uint32_t* b, const uint32_t* bias, uint32_t* out, uint32_t m,
                              uint32_t k, uint32_t n, cudaStream_t s);
cudaError_t launch_moe_gate(const float* scores, uint32_t* idx, float* weights, uint32_t tokens, uint32_t experts,
                            uint32_t k, cudaStream_t s);
cudaError_t launch_softmax_top_k(const float* scores, uint32_t* out_idx, float* out_w, float* best_vals,
                                 uint32_t* best_idxs, uint32_t n, uint32_t k, cudaStream_t s);
cudaError_t launch_top_k(const float* in, uint32_t* out_idx, float* best_vals, uint32_t* best_idxs, uint32_t n,
                         uint32_t k, cudaStream_t s);
cudaError_t launch_swiglu(const void* gate, const void* up, void* out, uint32_t n, uint32_t dtype, cudaStream_t s);
cudaError_t launch_residual_add(const void* residual, const void* branch, void* out, uint32_t n, uint32_t dtype, cudaStream_t s);
// learned_rms_norm (gate == nullptr) and gated_rms_norm; dtypes: 0 f32, 1 bf16, 2 f16; tree: the sum of squares as a
// two-level tree (kernel variant 8) instead of the reference's chain
cudaError_t launch_rms_norm(const void* input, const void* weight, const void* gate, void* out, uint32_t rows, uint32_t hidden,
                            float eps, uint32_t dtype, uint32_t weight_dtype, bool tree, cudaStream_t s);
// GGML K-quants with per-block f32 scale / min sidecars; bits = 4 (Q4_K) or 2 (Q2_K)
cudaError_t launch_k_quant_unpack(const uint32_t* packed, const float* scales, const float* mins, float* out, uint32_t n,
                                  uint32_t bits, cudaStream_t s);
// K-quant linear at size (dropin_fast.cu; kernel variant 7): out_dim a multiple of the outputs of four packed words; `partial`
// is scratch of k_quant_linear_fast_scratch_bytes(out_dim) bytes (one partial output row per k chunk)
constexpr uint32_t K_QUANT_K_CHUNKS = 64;
bool k_quant_linear_fast_supported(uint32_t in_dim, uint32_t out_dim, uint32_t bits);
size_t k_quant_linear_fast_scratch_bytes(uint32_t out_dim);
cudaError_t launch_k_quant_linear_fast(const float* x, const uint32_t* packed, const float* scales, const float* mins,
                                       const float* b, float* out, float* partial, uint32_t in_dim, uint32_t out_dim,
                                       uint32_t bits, int sm_count, cudaStream_t s);
cudaError_t launch_k_quant_linear(const float* x, const uint32_t* packed, const float* scales, const float* mins, const float* b,
                                  float* out, uint32_t in_dim, uint32_t out_dim, uint32_t bits, cudaStream_t s);
// hidden_scratch: f32 [hidden]
cudaError_t launch_expert_mlp(const float* x, const float* wg, const float* bg, const float* wu, const float* bu,
                              const float* wd, const float* bd, float* out, float* hidden_scratch, uint32_t in_dim,
                              uint32_t hidden, uint32_t out_dim, cudaStream_t s);
cudaError_t launch_moe_layer_accumulate(const float* weights, const float* expert_out, float* out, uint32_t k,
                                        uint32_t out_dim, cudaStream_t s);

}  // namespace vybk
