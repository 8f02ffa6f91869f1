// Device-side pieces shared by the kernels that gather over peer memory (allgather_push.cu, int4_gemv_halfsm.cu): where
// a rank's arrival counters live, and the bounded wait on them. Nothing here waits on another kernel of the same GPU.
#pragma once
#include <stdint.h>

#include "kernels.h"

namespace vybk {

constexpr long long PEER_WAIT_CLOCKS = 4000000000ll;  // about 2 s: the limit of a wait unless the context sets another
constexpr uint32_t PEER_COUNTER_STRIDE = 8;           // 32-bit words between the counters of two source ranks (one 32-byte sector each)

// local words of a context (PeerGather::epoch): [0, 8) pushes completed per peer slot, [8, 10) tickets,
// [10, 12) the launch index handed from one fused GEMV launch to the next (one word per buffer half), [12] a signal owed
constexpr uint32_t EPOCH_TICKET = 8, EPOCH_INDEX = 10, EPOCH_OWED = 12;
// [13] a slice that still has to be pushed to the peers (1 + its buffer half; 0: none), [14], [15] its batch rows and width
constexpr uint32_t EPOCH_PUSH = 13, EPOCH_PUSH_M = 14, EPOCH_PUSH_N = 15;

__device__ __forceinline__ const volatile uint32_t* counter_from(const PeerGather& ag, uint32_t owner, uint32_t source) {
    return reinterpret_cast<const volatile uint32_t*>(ag.peer_flag[owner]) + source * PEER_COUNTER_STRIDE;
}

// Has rank `source` completed `launches` pushes into this rank's buffer? Bounded; a wait that has run out once is not
// repeated: later calls return at once, so a broken run ends quickly with its status word set.
__device__ __forceinline__ bool wait_pushes_from(const PeerGather& ag, uint32_t source, uint32_t launches, const uint32_t* status) {
    if (status && (*reinterpret_cast<const volatile uint32_t*>(status) & 128u)) return false;
    const volatile uint32_t* arrived = counter_from(ag, ag.rank, source);
    const long long limit = ag.wait_clocks ? (long long)ag.wait_clocks : PEER_WAIT_CLOCKS;
    const long long t0 = clock64();
    while (int32_t(*arrived - launches) < 0) {
        if (clock64() - t0 > limit) return false;
        __nanosleep(64);
    }
    return true;
}

// A fused GEMV launch leaves its arrival signal to whatever runs next on the stream (the next fused launch or the wait
// kernel): by then the launch is complete and its peer stores are visible, so no CTA has to sit out a system-scope fence
// before the launch can end. Lanes 0..world-1 of one warp of ONE CTA call this.
__device__ __forceinline__ void send_owed_signal(const PeerGather& ag, uint32_t lane) {
    volatile uint32_t* owed = reinterpret_cast<volatile uint32_t*>(ag.epoch) + EPOCH_OWED;
    const bool pending = *owed != 0;
    __syncwarp();
    if (pending && lane < ag.world && lane != ag.rank)
        atomicAdd_system(const_cast<uint32_t*>(counter_from(ag, lane, ag.rank)), 1u);
    __syncwarp();
    if (lane == 0 && pending) *owed = 0;
}

}  // namespace vybk
