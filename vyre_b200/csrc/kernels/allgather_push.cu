// All-gather of column-parallel outputs over peer memory (NVLink), for one process per GPU.
//
// Every rank owns a gather buffer [2][world][m][n] bf16 (two halves, used alternately) that all ranks can address
// (symmetric memory). A plain GEMV writes rank r's [m, n] slice into the local buffer; the push kernel copies that
// slice into the same place of every peer's buffer with 16-byte stores, fences once at system scope, bumps every
// peer's 32-bit arrival counter and advances the local launch counter. Before it overwrites a half it checks
// (bounded) that every peer has completed all earlier pushes: then whatever consumed that half two steps ago has
// run, because consumers sit between a rank's launches in its stream. The wait kernel is the consumer-side check:
// every gather started so far on this rank is complete in local memory. All waits are clock-bounded (~2 s) and raise
// status bit 128 instead of hanging. Nothing here waits on another kernel of the same GPU, and no multicast is used.
//
// The reference's backends are single-device; the sharding follows from its one-output-per-invocation kernels
// (vyre-libs/src/nn/linear/inner/linear_4bit.rs:710-742).
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace vybk {
namespace {

constexpr long long WAIT_CLOCKS = 4000000000ll;

// a wait that has run out once is not repeated: later calls return at once, so a broken run ends quickly with its
// status word set instead of spending the clock limit on every launch
__device__ __forceinline__ bool wait_arrivals(const PeerGather& ag, uint32_t launches, const uint32_t* status) {
    if (ag.world <= 1) return true;
    if (status && (*reinterpret_cast<const volatile uint32_t*>(status) & 128u)) return false;
    const volatile uint32_t* arrived = reinterpret_cast<const volatile uint32_t*>(ag.peer_flag[ag.rank]);
    const uint32_t want = launches * (ag.world - 1);
    const long long t0 = clock64();
    while (int32_t(*arrived - want) < 0) {
        if (clock64() - t0 > WAIT_CLOCKS) return false;
        __nanosleep(64);
    }
    return true;
}

__global__ void __launch_bounds__(256) allgather_push_kernel(const PeerGather ag, uint32_t half, uint32_t m, uint32_t n,
                                                             uint32_t* status) {
    __shared__ uint32_t s_epoch;
    if (threadIdx.x == 0) {
        const uint32_t done = *reinterpret_cast<const volatile uint32_t*>(ag.epoch);
        s_epoch = done;
        if (!wait_arrivals(ag, done, status) && status) atomicOr(status, 128u);
    }
    __syncthreads();
    const size_t slice_vecs = size_t(m) * n * 2 / 16;
    const size_t slice_off = (size_t(half) * ag.world + ag.rank) * slice_vecs;
    const uint4* src = reinterpret_cast<const uint4*>(ag.peer_out[ag.rank]) + slice_off;
    for (uint32_t r = 0; r < ag.world; ++r) {
        if (r == ag.rank) continue;
        uint4* dst = reinterpret_cast<uint4*>(ag.peer_out[r]) + slice_off;
        for (size_t i = threadIdx.x; i < slice_vecs; i += blockDim.x) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t r = 0; r < ag.world; ++r)
            if (r != ag.rank) atomicAdd_system(reinterpret_cast<unsigned int*>(ag.peer_flag[r]), 1u);
        *reinterpret_cast<volatile uint32_t*>(ag.epoch) = s_epoch + 1;
    }
}

__global__ void __launch_bounds__(32) allgather_wait_kernel(const PeerGather ag, uint32_t* status) {
    if (threadIdx.x != 0) return;
    const uint32_t done = *reinterpret_cast<const volatile uint32_t*>(ag.epoch);
    const bool ok = wait_arrivals(ag, done, status);
    __threadfence_system();  // acquire side: the peers' stores are visible to whatever follows in this stream
    if (!ok && status) atomicOr(status, 128u);
}

}  // namespace

cudaError_t launch_allgather_push(const PeerGather& ag, uint32_t half, uint32_t m, uint32_t n, cudaStream_t stream,
                                  uint32_t* status) {
    if (ag.world < 1 || ag.world > 8 || ag.rank >= ag.world || half > 1 || (size_t(m) * n) % 8) return cudaErrorInvalidValue;
    allgather_push_kernel<<<1, 256, 0, stream>>>(ag, half, m, n, status);
    return cudaGetLastError();
}

cudaError_t launch_allgather_wait(const PeerGather& ag, cudaStream_t stream, uint32_t* status) {
    if (ag.world < 1 || ag.world > 8 || ag.rank >= ag.world) return cudaErrorInvalidValue;
    allgather_wait_kernel<<<1, 32, 0, stream>>>(ag, status);
    return cudaGetLastError();
}

}  // namespace vybk
