// All-gather of column-parallel outputs over peer memory (NVLink), for one process per GPU.
//
// Every rank owns a gather buffer [2][world][m][n] bf16 (two halves, used alternately) that all ranks can address
// (symmetric memory), and eight 32-bit arrival counters, one per source rank. A plain GEMV writes rank r's [m, n]
// slice into the local buffer; the push kernel runs ONE CTA PER PEER: it copies that slice into the same place of
// its peer's buffer with 16-byte stores, fences at system scope and bumps the peer's counter for this rank. The
// peers are served side by side, so the cost of a push does not grow with the number of ranks. Before a CTA
// overwrites a half on its peer it checks (bounded) that this peer has completed as many pushes as this rank has:
// then whatever consumed that half two steps ago on the peer has run, because consumers sit between a rank's
// launches in its stream. The wait kernel is the consumer-side check: every gather started so far on this rank is
// complete in local memory. All waits are clock-bounded (about 2 s unless the context sets another limit) and
// raise status bit 128 instead of hanging; a wait that has run out once is not repeated. Nothing here waits on
// another kernel of the same GPU, and no multicast is used.
//
// The reference's backends are single-device; the sharding follows from its one-output-per-invocation kernels
// (vyre-libs/src/nn/linear/inner/linear_4bit.rs:710-742).
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"
#include "peer_gather.cuh"

namespace vybk {
namespace {

// One CTA per peer, and a small one: 128 threads at no more than 32 registers and a few bytes of shared memory, so that
// it becomes resident BESIDE the two decode-GEMV CTAs an SM holds under programmatic dependent launch (those take 512
// threads, 61440 of the 65536 registers and all but 4 KB of the shared memory). A larger push CTA would have to wait for
// a GEMV CTA to leave, or the GEMV would have to keep an SM free and lose the pairing of consecutive launches on it.
__global__ void __launch_bounds__(128, 16) allgather_push_kernel(const PeerGather ag, uint32_t half, uint32_t m, uint32_t n,
                                                             uint32_t* status) {
    const uint32_t peer = blockIdx.x < ag.rank ? blockIdx.x : blockIdx.x + 1;
    volatile uint32_t* my_epoch = reinterpret_cast<volatile uint32_t*>(ag.epoch) + blockIdx.x;  // pushes this CTA slot has done
    __shared__ uint32_t s_done;
    if (threadIdx.x == 0) {
        s_done = *my_epoch;
        // with two halves: the peer has completed every push this rank has; with more slots the same minus the slots
        // that separate this push from the last one into the same slot
        const uint32_t slack = ag.slots > 2 ? uint32_t(ag.slots) - 2u : 0u;
        if (s_done > slack && !wait_pushes_from(ag, peer, s_done - slack, status) && status) atomicOr(status, 128u);
    }
    __syncthreads();
    const size_t slice_vecs = size_t(m) * n * 2 / 16;
    const size_t slice_off = (size_t(half) * ag.world + ag.rank) * slice_vecs;
    const uint4* src = reinterpret_cast<const uint4*>(ag.peer_out[ag.rank]) + slice_off;
    uint4* dst = reinterpret_cast<uint4*>(ag.peer_out[peer]) + slice_off;
    for (size_t i = threadIdx.x; i < slice_vecs; i += blockDim.x) dst[i] = src[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        atomicAdd_system(const_cast<uint32_t*>(counter_from(ag, peer, ag.rank)), 1u);
        atomicAdd(const_cast<uint32_t*>(my_epoch), 1u);  // pushes of several streams may run side by side
    }
}

__global__ void __launch_bounds__(256) allgather_wait_kernel(const PeerGather ag, uint32_t* status) {
    volatile uint32_t* e = reinterpret_cast<volatile uint32_t*>(ag.epoch);
    if (threadIdx.x < 32) send_owed_signal(ag, threadIdx.x);  // of a fused GEMV launch before this kernel in the stream
    const uint32_t done = e[0];
    const uint32_t pending = e[EPOCH_PUSH];
    __syncthreads();
    if (pending != 0) {
        // the last launch of a pipelined chain left its slice in local memory: carry it to the peers and signal it
        bool fine = true;
        if (threadIdx.x < ag.world && threadIdx.x != ag.rank && done >= 2) fine = wait_pushes_from(ag, threadIdx.x, done - 2, status);
        if (!fine && status) atomicOr(status, 128u);
        __syncthreads();
        const size_t elems = size_t(e[EPOCH_PUSH_M]) * e[EPOCH_PUSH_N];
        const size_t base = (size_t(pending - 1) * ag.world + ag.rank) * elems;
        const uint16_t* src = reinterpret_cast<const uint16_t*>(ag.peer_out[ag.rank]) + base;
        for (size_t i = threadIdx.x; i < elems; i += blockDim.x) {
            const uint16_t v = src[i];
            for (uint32_t q = 0; q < ag.world; ++q)
                if (q != ag.rank) reinterpret_cast<uint16_t*>(ag.peer_out[q])[base + i] = v;
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < ag.world && threadIdx.x != ag.rank)
            atomicAdd_system(const_cast<uint32_t*>(counter_from(ag, threadIdx.x, ag.rank)), 1u);
        if (threadIdx.x == 0) e[EPOCH_PUSH] = 0;
    }
    bool ok = true;
    if (threadIdx.x < ag.world && threadIdx.x != ag.rank) ok = wait_pushes_from(ag, threadIdx.x, done, status);
    __threadfence_system();  // acquire side: the peers' stores are visible to whatever follows in this stream
    if (!ok && status) atomicOr(status, 128u);
}

// ---- column-parallel gather of a row block: every rank's [rows, local columns] block lands at its column offset of
// every rank's [M, N] buffer (own rank included). `per_dest` CTAs per destination share the rows (enough of them to
// keep a few hundred KB in flight towards every destination); the last of them to finish (a ticket in local memory)
// fences and bumps the destination's counter for this rank, once per call.
__global__ void __launch_bounds__(256)
colpar_push_kernel(const PeerGather ag, const uint4* __restrict__ src, uint32_t rows, uint32_t row_vecs, uint64_t dst_pitch_vecs,
                   uint64_t dst_off_vecs, uint32_t per_dest, uint32_t* tickets, uint32_t* status) {
    const uint32_t dest = blockIdx.x / per_dest, part = blockIdx.x % per_dest;
    uint4* dst = reinterpret_cast<uint4*>(ag.peer_out[dest]) + dst_off_vecs;
    // 16-byte vectors of the block, spread over the CTAs of this destination row by row, four loads in flight per thread
    for (uint32_t r = part; r < rows; r += per_dest) {
        const uint4* s = src + size_t(r) * row_vecs;
        uint4* d = dst + size_t(r) * dst_pitch_vecs;
        uint32_t i = threadIdx.x;
        for (; i + 3 * 256 < row_vecs; i += 4 * 256) {
            const uint4 a = s[i], b = s[i + 256], c = s[i + 512], e = s[i + 768];
            d[i] = a;
            d[i + 256] = b;
            d[i + 512] = c;
            d[i + 768] = e;
        }
        for (; i < row_vecs; i += 256) d[i] = s[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(&tickets[dest], 1u) == per_dest - 1) {
            tickets[dest] = 0;  // the next call finds it clear (calls are ordered by the stream)
            __threadfence_system();
            atomicAdd_system(const_cast<uint32_t*>(counter_from(ag, dest, ag.rank)), 1u);
        }
    }
    (void)status;
}

// After a gathering GEMM (whose epilogue stored this rank's block into every rank's output): one more block delivered
// everywhere. Runs after that GEMM in its stream, so the block is complete and visible; one thread per destination.
__global__ void __launch_bounds__(32) colpar_signal_kernel(const PeerGather ag) {
    if (threadIdx.x < ag.world) {
        __threadfence_system();
        atomicAdd_system(const_cast<uint32_t*>(counter_from(ag, threadIdx.x, ag.rank)), 1u);
    }
}

// bounded wait until every rank (own included) has delivered `want` blocks into this rank's buffer
__global__ void __launch_bounds__(32) colpar_wait_kernel(const PeerGather ag, uint32_t want, uint32_t* status) {
    bool ok = true;
    if (threadIdx.x < ag.world) ok = wait_pushes_from(ag, threadIdx.x, want, status);
    __threadfence_system();
    if (!ok && status) atomicOr(status, 128u);
}

}  // namespace

cudaError_t launch_colpar_push(const PeerGather& ag, const void* src, uint32_t rows, uint32_t row_bytes, uint64_t dst_pitch_bytes,
                               uint64_t dst_offset_bytes, uint32_t* tickets, cudaStream_t stream, uint32_t* status) {
    if (ag.world < 1 || ag.world > 8 || ag.rank >= ag.world || (row_bytes | dst_pitch_bytes | dst_offset_bytes) % 16 ||
        (reinterpret_cast<uintptr_t>(src) & 15) || !tickets)
        return cudaErrorInvalidValue;
    if (rows == 0) return cudaSuccess;
    // one CTA per 64 KB of the block and destination, at most 592 CTAs in all (four per SM)
    const uint64_t bytes = uint64_t(rows) * row_bytes;
    uint32_t per_dest = uint32_t((bytes + 65535) / 65536);
    const uint32_t cap = 592u / ag.world;
    per_dest = per_dest < 1 ? 1 : per_dest > cap ? cap : per_dest;
    if (per_dest > rows) per_dest = rows;
    colpar_push_kernel<<<ag.world * per_dest, 256, 0, stream>>>(ag, static_cast<const uint4*>(src), rows, row_bytes / 16,
                                                                 dst_pitch_bytes / 16, dst_offset_bytes / 16, per_dest, tickets, status);
    return cudaGetLastError();
}

cudaError_t launch_colpar_signal(const PeerGather& ag, cudaStream_t stream) {
    if (ag.world < 1 || ag.world > 8 || ag.rank >= ag.world) return cudaErrorInvalidValue;
    colpar_signal_kernel<<<1, 32, 0, stream>>>(ag);
    return cudaGetLastError();
}

cudaError_t launch_colpar_wait(const PeerGather& ag, uint32_t want, cudaStream_t stream, uint32_t* status) {
    if (ag.world < 1 || ag.world > 8 || ag.rank >= ag.world) return cudaErrorInvalidValue;
    colpar_wait_kernel<<<1, 32, 0, stream>>>(ag, want, status);
    return cudaGetLastError();
}

cudaError_t launch_allgather_push(const PeerGather& ag, uint32_t half, uint32_t m, uint32_t n, cudaStream_t stream,
                                  uint32_t* status) {
    if (ag.world < 1 || ag.world > 8 || ag.rank >= ag.world || half >= (ag.slots ? ag.slots : 2) || (size_t(m) * n) % 8) return cudaErrorInvalidValue;
    if (ag.world == 1) return cudaSuccess;  // nobody to send to
    allgather_push_kernel<<<ag.world - 1, 128, 0, stream>>>(ag, half, m, n, status);
    return cudaGetLastError();
}

cudaError_t launch_allgather_wait(const PeerGather& ag, cudaStream_t stream, uint32_t* status) {
    if (ag.world < 1 || ag.world > 8 || ag.rank >= ag.world) return cudaErrorInvalidValue;
    allgather_wait_kernel<<<1, 256, 0, stream>>>(ag, status);
    return cudaGetLastError();
}

}  // namespace vybk
