// One-shot allreduce of a short F32 vector over NVLink peer memory (no reference analogue: the
// reference is single-device). A decode step of the row-split layer stack sums a 20 KB vector over
// the ranks 128 times per token; at that size a collective is pure latency, and a library call
// costs ~20 us. This kernel costs one peer store and a local sum.
//
// Every rank owns an inbox in its own memory: [2 parities][ranks][capacity] words of 8 bytes, each
// a float beside a 32-bit tag. A call with sequence number s uses parity s & 1 and tag s + 1 (never 0):
//   1. each rank stores (value, tag) for every element into slot [parity][its rank] of every
//      peer's inbox: plain peer stores, so remote data is always written into the consumer's own
//      memory and never loaded from a peer. An 8-byte store is single-copy atomic, so a reader
//      that sees the tag sees the value: no fence and no separate flag are needed;
//   2. it polls its own inbox, with a bound, until every peer's word carries the tag;
//   3. it adds the values in rank order (every rank adds the same numbers in the same order, so
//      all ranks hold bit-identical sums) and writes the result over its vector.
// Two parities suffice: a rank can be at most one call ahead of a peer, because finishing call
// s + 1 needs the peer's words for s + 1, which the peer sends only after its kernel for call s
// has ended; so words of call s + 2 (same parity as s) never land on words a peer still reads.
// The sequence number lives in device memory (a replayed graph cannot change kernel arguments);
// the last block to finish advances it. Threads work on disjoint elements; nothing waits on
// another thread of the same grid.
// A wait is bounded both by iterations and by the global timer (two seconds unless the host set another
// limit: ranks replay their graphs from separate processes, so a peer may legitimately arrive late by a
// host hiccup).
// When it runs out the block raises the backend's status word, sets a sticky local word that makes
// every later call return at once, and returns; the host reports the failure at commit.
#include "kernels.hpp"

namespace nu {

constexpr uint32_t kPushSpinLimit = 1u << 24;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void store_words(uint4 *dst, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 load_words(const uint4 *src) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
    return v;
}

template <bool PUSH>
__global__ void __launch_bounds__(256) push_allreduce_kernel(PushParams p) {
    // The kernel after this one may start its prologue now; this one reads the vector only after
    // the kernel before it has ended.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t tid = threadIdx.x;
    // p.seq: [0] sequence number, [1] blocks finished in this call, [2] sticky failure
    __shared__ uint32_t head[2];
    if (tid == 0) {
        head[0] = *(volatile uint32_t *)(p.seq + 2);
        head[1] = *(volatile uint32_t *)p.seq;
    }
    __syncthreads();
    if (head[0] != 0) {  // uniform over the block
        if (tid == 0) atomicExch(p.status, 2u);
        return;
    }
    const uint32_t seq = head[1];
    const uint32_t parity = seq & 1u, tag = push_tag(seq);
    const uint32_t pairs = (p.count + 1) / 2;  // a thread moves two elements: one 16-byte word pair
    const uint32_t first = blockIdx.x * blockDim.x + tid, step = gridDim.x * blockDim.x;
    // The sequence number is 32 bits wide and wraps after some 23 hours of decoding. A word that no call has
    // rewritten for a whole period (the tail of a slot, beyond the longest vector summed lately) could then
    // carry the tag of a new call. So twice per 2^30 calls (once per parity) a rank clears the tails of its
    // own slots of this parity: no peer writes there during this call (a peer is at most one call ahead, on
    // the other parity), and afterwards no word of the inbox is older than 2^30 calls.
    if (((seq >> 1) & 0x1fffffffu) == 0u) {
        const uint32_t cap_pairs = p.capacity / 2;
        for (uint32_t r = 0; r < p.ranks; ++r)
            for (uint32_t i = pairs + first; i < cap_pairs; i += step)
                store_words((uint4 *)(p.inbox[p.rank] + ((size_t)parity * p.ranks + r) * p.capacity) + i, make_uint4(0u, 0u, 0u, 0u));
    }
    // ---- 1. push (not when the producer of the vector pushed it already, into this rank's inbox too) ----
    for (uint32_t i = first; PUSH && i < pairs; i += step) {
        const float a = p.buf[2 * i], b = 2 * i + 1 < p.count ? p.buf[2 * i + 1] : 0.0f;
        const uint4 w = make_uint4(__float_as_uint(a), tag, __float_as_uint(b), tag);
        for (uint32_t r = 0; r < p.ranks; ++r)
            if (r != p.rank) store_words((uint4 *)(p.inbox[r] + ((size_t)parity * p.ranks + p.rank) * p.capacity) + i, w);
    }
    // ---- 2, 3. poll my inbox and add in rank order ----
    const unsigned long long t0 = global_ns();
    bool failed = false;
    for (uint32_t i = first; i < pairs && !failed; i += step) {
        const bool both = 2 * i + 1 < p.count;  // the last word pair of an odd count has one element
        // all ranks' words are requested at once (eight dependent round trips to L2 would be the whole latency of the
        // call at eight ranks); then each is polled until it carries the tag
        uint4 w[PUSH_MAX_RANKS];
#pragma unroll
        for (int r = 0; r < PUSH_MAX_RANKS; ++r)
            if ((uint32_t)r < p.ranks && !(PUSH && (uint32_t)r == p.rank))
                w[r] = load_words((const uint4 *)(p.inbox[p.rank] + ((size_t)parity * p.ranks + r) * p.capacity) + i);
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int r = 0; r < PUSH_MAX_RANKS; ++r) {
            if ((uint32_t)r >= p.ranks || failed) continue;
            float a, b;
            if (PUSH && (uint32_t)r == p.rank) {
                a = p.buf[2 * i];
                b = both ? p.buf[2 * i + 1] : 0.0f;
            } else {
                const uint4 *src = (const uint4 *)(p.inbox[p.rank] + ((size_t)parity * p.ranks + r) * p.capacity) + i;
                uint32_t n = 0;
                while ((w[r].y != tag || (both && w[r].w != tag)) && ++n < kPushSpinLimit) {
                    if ((n & 255u) == 0 && global_ns() - t0 > p.wait_ns) break;
                    w[r] = load_words(src);
                }
                if (w[r].y != tag || (both && w[r].w != tag)) { failed = true; continue; }
                a = __uint_as_float(w[r].x);
                b = both ? __uint_as_float(w[r].z) : 0.0f;
            }
            if (r == 0) { s0 = a; s1 = b; }
            else { s0 += a; s1 += b; }
        }
        if (!failed) {
            if (p.add_to) {
                // the residual add behind the projection whose outputs were summed: every rank adds the same sum to the same residual
                p.add_to[2 * i] += s0;
                if (both) p.add_to[2 * i + 1] += s1;
            } else {
                p.buf[2 * i] = s0;
                if (both) p.buf[2 * i + 1] = s1;
            }
        }
    }
    if (__syncthreads_or(failed)) {
        if (tid == 0) {
            atomicExch(p.status, 2u);
            atomicExch(p.seq + 2, 1u);
        }
        return;
    }
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
    const uint32_t pairs = (p.count + 1) / 2;
    uint32_t blocks = (pairs + 255) / 256;
    if (blocks > PUSH_MAX_BLOCKS) blocks = PUSH_MAX_BLOCKS;
    if (blocks == 0) blocks = 1;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, push_allreduce_kernel<true>, p);
    return 1;
}

int launch_gather_sum(cudaStream_t s, const PushParams &p) {
    const uint32_t pairs = (p.count + 1) / 2;
    uint32_t blocks = (pairs + 255) / 256;
    if (blocks > PUSH_MAX_BLOCKS) blocks = PUSH_MAX_BLOCKS;
    if (blocks == 0) blocks = 1;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, push_allreduce_kernel<false>, p);
    return 1;
}

}  // namespace nu
