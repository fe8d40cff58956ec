// One-shot allreduce of a short F32 vector over NVLink peer memory (no reference analogue: the
// reference is single-device). A decode step of the row-split layer stack sums a 20 KB vector over
// the ranks 128 times per token; at that size a collective is pure latency, and a library call
// costs ~20-30 us. This kernel costs a peer store, a flag and a local sum.
//
// Every rank owns an inbox in its own memory: [2 parities][ranks][capacity] floats and, per block
// of the grid, a flag per (parity, source rank). A call with sequence number s uses parity s & 1:
//   1. each rank stores its vector into slot [parity][my rank] of every peer's inbox (plain peer
//      stores: remote data is always written into the consumer's own memory, never loaded from a peer);
//   2. after a system-scope fence it stores s + 1 into its flag in every peer's inbox;
//   3. it waits, with a bound, until the flags of all peers in its own inbox show s + 1;
//   4. it adds the slots in rank order (every rank adds the same numbers in the same order, so all
//      ranks hold bit-identical sums) and writes the result over its vector.
// Two parities suffice: a rank can be at most one call ahead of a peer, because finishing call
// s + 1 needs the peer's flags for s + 1, which the peer sends only after its kernel for call s has
// ended. Blocks of the grid work on disjoint slices with their own flags; no block waits on
// another block of the same grid. The sequence number lives in device memory (a replayed graph
// cannot change kernel arguments); the last block to finish advances it.
// A wait is bounded both by iterations and by the global timer (about two seconds: ranks replay
// their graphs from separate processes, so a peer may legitimately arrive late by a host hiccup).
// When it runs out the block raises the backend's status word, sets a sticky local word that makes
// every later call return at once, and returns; the host reports the failure at commit.
#include "kernels.hpp"

namespace nu {

constexpr uint32_t kPushSpinLimit = 1u << 24;
constexpr unsigned long long kPushWaitNs = 2000000000ull;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(256) push_allreduce_kernel(PushParams p) {
    const uint32_t b = blockIdx.x, tid = threadIdx.x;
    const uint32_t per = ((p.count + gridDim.x - 1) / gridDim.x + 3u) & ~3u;  // slice, a multiple of 4 floats
    const uint32_t c0 = min(b * per, p.count), c1 = min(c0 + per, p.count);
    // p.seq: [0] sequence number, [1] blocks finished in this call, [2] sticky failure
    if (*(volatile uint32_t *)(p.seq + 2) != 0) {
        if (tid == 0) atomicExch(p.status, 2u);
        return;
    }
    const uint32_t seq = *(volatile uint32_t *)p.seq;
    const uint32_t parity = seq & 1u;
    const size_t slot_floats = p.capacity;
    // ---- 1. push my slice into every peer's inbox (and my own) ----
    for (uint32_t r = 0; r < p.ranks; ++r) {
        float *dst = p.inbox[r] + ((size_t)parity * p.ranks + p.rank) * slot_floats;
        for (uint32_t i = c0 + tid * 4; i < c1; i += blockDim.x * 4) {
            if (i + 4 <= c1) *(float4 *)(dst + i) = *(const float4 *)(p.buf + i);
            else for (uint32_t j = i; j < c1; ++j) dst[j] = p.buf[j];
        }
    }
    __threadfence_system();
    __syncthreads();
    // ---- 2. flags ----
    if (tid < p.ranks) {
        volatile uint32_t *flag = p.flags[tid] + ((size_t)parity * p.ranks + p.rank) * PUSH_MAX_BLOCKS + b;
        *flag = seq + 1;
    }
    // ---- 3. wait for every rank's flag in my inbox ----
    __shared__ uint32_t failed;
    if (tid == 0) failed = 0;
    __syncthreads();
    if (tid < p.ranks) {
        volatile uint32_t *flag = p.flags[p.rank] + ((size_t)parity * p.ranks + tid) * PUSH_MAX_BLOCKS + b;
        const unsigned long long t0 = global_ns();
        uint32_t i = 0;
        bool ok = false;
        while (!(ok = (*flag == seq + 1)) && ++i < kPushSpinLimit)
            if ((i & 1023u) == 0 && global_ns() - t0 > kPushWaitNs) break;
        if (!ok) failed = 1;
    }
    __syncthreads();
    if (failed) {
        if (tid == 0) {
            atomicExch(p.status, 2u);
            atomicExch(p.seq + 2, 1u);
        }
        return;
    }
    __threadfence_system();
    // ---- 4. add the slots in rank order ----
    const float *mine = p.inbox[p.rank] + (size_t)parity * p.ranks * slot_floats;
    for (uint32_t i = c0 + tid * 4; i < c1; i += blockDim.x * 4) {
        if (i + 4 <= c1) {
            float4 s = __ldcg((const float4 *)(mine + i));
            for (uint32_t r = 1; r < p.ranks; ++r) {
                const float4 v = __ldcg((const float4 *)(mine + r * slot_floats + i));
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            *(float4 *)(p.buf + i) = s;
        } else {
            for (uint32_t j = i; j < c1; ++j) {
                float s = __ldcg(mine + j);
                for (uint32_t r = 1; r < p.ranks; ++r) s += __ldcg(mine + r * slot_floats + j);
                p.buf[j] = s;
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(p.seq + 1, 1u) == gridDim.x - 1) {
            p.seq[1] = 0;
            __threadfence();
            *(volatile uint32_t *)p.seq = seq + 1;
        }
    }
}

int launch_push_allreduce(cudaStream_t s, const PushParams &p) {
    uint32_t blocks = (p.count + 2047) / 2048;
    if (blocks > PUSH_MAX_BLOCKS) blocks = PUSH_MAX_BLOCKS;
    if (blocks == 0) blocks = 1;
    push_allreduce_kernel<<<blocks, 256, 0, s>>>(p);
    return 1;
}

}  // namespace nu
