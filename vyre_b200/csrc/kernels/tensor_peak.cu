// Tensor-core peak microbenchmark: tcgen05.mma from operands that never leave shared memory.
//
// The roofline of the int8 x int8 -> int32 GEMM needs a denominator, and no measured int8 peak exists for the pool
// (the driver measures a cuBLAS bf16 GEMM only). This kernel gives one: every CTA (one per SM) allocates tensor
// memory, points two shared-memory descriptors at a fixed 128 x 128-byte A tile and a 256 x 128-byte B tile, and one
// thread issues `iters` rounds of four MMAs (128 x 256 x 32 each for 8-bit operands, 128 x 256 x 16 for bf16) into two
// alternating accumulators. No loads, no epilogue: what is timed is the MMA pipe itself, with the same instruction
// shape the GEMM uses. The operand bytes are whatever shared memory holds after a zero fill (the pipe's speed does
// not depend on the values; the power draw does, so the figure is an upper bound for real data).
//
// Used by bench.py only. Every wait is bounded.
#include "kernels.h"
#include "tcgen05_common.cuh"

namespace vybk {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 256, BK_BYTES = 128;
constexpr int A_BYTES = BM * BK_BYTES, B_BYTES = BN * BK_BYTES;
constexpr int SMEM_BYTES = A_BYTES + B_BYTES + 1024 + 64;

template <bool INT8>
__global__ void __launch_bounds__(128, 1) tensor_peak_kernel(uint32_t iters, uint32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned long long* bar = reinterpret_cast<unsigned long long*>(tiles + A_BYTES + B_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
    volatile unsigned int* abort_flag = reinterpret_cast<volatile unsigned int*>(bar + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 16; i += blockDim.x) reinterpret_cast<uint4*>(tiles)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(bar), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (warp == 0) {
        if (lane == 0) {
            const uint64_t da = smem_desc_sw128(smem_u32(tiles)), db = smem_desc_sw128(smem_u32(tiles + A_BYTES));
            constexpr uint32_t idesc = INT8 ? idesc_s8_s32(BM, BN) : idesc_bf16_f32(BM, BN);
            for (uint32_t it = 0; it < iters; ++it) {
                const uint32_t d = tmem_base + (it & 1u) * BN;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if constexpr (INT8)
                        mma_i8(d, smem_desc_advance(da, k * 32), smem_desc_advance(db, k * 32), idesc, 1u);
                    else
                        mma_f16(d, smem_desc_advance(da, k * 32), smem_desc_advance(db, k * 32), idesc, 1u);
                }
            }
            tc_commit(smem_u32(bar));
        }
        __syncwarp();
        bool ok = mbar_wait(smem_u32(bar), 0, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok && lane == 0 && status) atomicOr(status, 8u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace

cudaError_t launch_tensor_peak(uint32_t int8, uint32_t iters, int sm_count, cudaStream_t stream, uint32_t* status,
                               double* ops_per_launch) {
    cudaError_t e = int8 ? cudaFuncSetAttribute(tensor_peak_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES)
                         : cudaFuncSetAttribute(tensor_peak_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    // multiply-adds count twice; an 8-bit MMA covers 32 k, a bf16 one 16
    if (ops_per_launch) *ops_per_launch = 2.0 * BM * BN * (int8 ? 32.0 : 16.0) * 4.0 * double(iters) * double(sm_count);
    if (int8)
        tensor_peak_kernel<true><<<sm_count, 128, SMEM_BYTES, stream>>>(iters, status);
    else
        tensor_peak_kernel<false><<<sm_count, 128, SMEM_BYTES, stream>>>(iters, status);
    return cudaGetLastError();
}

}  // namespace vybk
