// A chain of one-token GEMV operators as ONE persistent launch: the decode step of a dense model is a
// string of matvecs, each reading what the one before wrote (QKV -> O -> gate/up pair -> down, layer after
// layer; inference/src/models/qwen35_metal.zig:589-640 records them one by one into a command buffer).
// As kernels of their own each of them pays for its launch, for the staging of its input by every block,
// for the ramp of its weight stream and for its tail, during all of which HBM idles: about a third of
// the step. Here one block per multiprocessor walks the whole list of operators:
//
//   for each operator:   re-make the slot barriers, start the weight stream of THIS operator (weights are
//                        constants, so this needs nothing from the operator before),
//                        wait until every block has finished the operator before (one arrival counter in
//                        global memory, acquire / release, bounded),
//                        stage the input rows, run the units (i8_kernel.cuh), publish the outputs, arrive.
//
// So while the slowest block still finishes operator i, the other blocks already have the first stages of
// operator i + 1 in flight (about 120 KB per multiprocessor), and the memory system never drains between two
// operators. All blocks must be resident at once: the grid is one block per multiprocessor and the kernel
// is launched cooperatively, which fails loudly instead of dead-locking if that cannot be had.
//
// Measured on a B200 (64-layer 27B-shape stack, one token): 225 tokens/s chained against 289 with a kernel per
// operator. In-kernel timers put a chained operator's fixed cost at 7 to 8 us (leaving the operator before and
// entering this one 1.3, barriers and first copies 1.1, waiting for the slowest block 1 to 2, staging 1.9, first
// task 1.3, the unit's sums 1.2) against about 3.5 us for a kernel of its own launched under the tail of the one
// before it. The chain is therefore opt-in (Backend::chaining); it stays as the measured alternative and as the
// frame for operators that must wait on other devices inside one launch.
//
// The operators may mix encodings and geometries (Q4_K: 4 slots x 5 parts, planar Q6_K: 6 x 3); the block
// has as many warps as the widest needs and the others idle through the narrower ones.
#include "i8_q4k.cuh"
#include "i8_q6k.cuh"

namespace nu {
namespace i8 {

constexpr int kChainThreads = Q4KPlain::THREADS > Q6KPlain::THREADS ? Q4KPlain::THREADS : Q6KPlain::THREADS;

enum : uint32_t { CHAIN_Q4K = 0, CHAIN_Q6K = 1 };

struct ChainOp {
    Params p;
    uint32_t kind, stages, grid, slots;
};
struct ChainParams {
    uint32_t count;
    uint32_t *arrivals;  // [0]: blocks that finished an operator; [1]: blocks that left the kernel. Both zero between launches.
    ChainOp op[kChainMax];
};
static_assert(sizeof(ChainParams) <= 32764, "kernel parameters are at most 32,764 bytes");

// Not inlined: each operator body keeps the register allocation it has as a kernel of its own.
// p: a copy of the operator's parameters in shared memory (as a callee this code cannot know that the kernel's
// parameter space never changes and would read it again after every wait); pm: the parameter space, for the tensor maps.
template <class E, class G, int STAGES>
__device__ __noinline__ void run_link(const Params *p, const Params *pm, uint8_t *smem, ChainLink link) {
    run_op<E, G, 1, (G::SLOTS >= 5)>(*p, *pm, STAGES, smem, link);  // shared units where a block has many slots (the plan may assume either)
}
template <class E, class G>
__device__ __forceinline__ void run_stages(const Params *p, const Params *pm, uint32_t stages, uint8_t *smem, const ChainLink &link) {
    switch (stages) {
    case 5: run_link<E, G, 5>(p, pm, smem, link); break;
    case 4: run_link<E, G, 4>(p, pm, smem, link); break;
    case 3: run_link<E, G, 3>(p, pm, smem, link); break;
    default: run_link<E, G, 2>(p, pm, smem, link); break;
    }
}
// Copies the scalar part of an operator's parameters (everything after the tensor maps) into shared memory.
__device__ __forceinline__ void stash_params(const Params &src, uint8_t *dst, uint32_t tid) {
    constexpr uint32_t FROM = offsetof(Params, out) / 16, TO = sizeof(Params) / 16;
    static_assert(offsetof(Params, out) % 16 == 0, "the scalars start on a 16-byte boundary");
    if (tid >= FROM && tid < TO) ((uint4 *)dst)[tid] = ((const uint4 *)&src)[tid];
}

__global__ void __launch_bounds__(kChainThreads, 1) chain_kernel(const __grid_constant__ ChainParams c) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t tid = threadIdx.x;
    asm volatile("griddepcontrol.launch_dependents;");
    uint32_t prev_slots = 0, prev_stages = 0;
    stash_params(c.op[0].p, smem + kParamsAt, tid);
    for (uint32_t i = 0; i < c.count; ++i) {
        const ChainOp &o = c.op[i];
        __syncthreads();  // every warp has left the operator before: its outputs are written, its stages, barriers and parameters are free
        // (not thread 0, which starts the weight stream of its slot next and should not sit out the fence)
        if (i && tid == kChainThreads - 32) {
            __threadfence();
            atomicAdd(c.arrivals, 1u);
        }
        // the copy engine's first use of a tensor map fetches it: have the next operator's maps on their way
        if (i + 1 < c.count && tid >= 32 && tid < 40) {
            const ChainOp &nx = c.op[i + 1];
            const uint32_t k = tid - 32;
            if ((k & 3u) < nx.p.count && (k < 4 || nx.kind == CHAIN_Q6K))
                asm volatile("prefetch.tensormap [%0];" ::"l"(k < 4 ? &nx.p.map[k] : &nx.p.map2[k & 3u]) : "memory");
        }
        // the next operator's parameters go to the copy the operator before used; the sync above of the next round publishes them
        if (i + 1 < c.count) stash_params(c.op[i + 1].p, smem + kParamsAt + ((i + 1) & 1u) * sizeof(Params), tid);
        const Params *ps = (const Params *)(smem + kParamsAt + (i & 1u) * sizeof(Params));
        const ChainLink link{c.arrivals, i * gridDim.x, prev_slots, prev_stages};
        if (blockIdx.x < o.grid) {
            if (o.kind == CHAIN_Q4K) {
                if (tid < (uint32_t)Q4KPlain::THREADS) run_stages<Q4K, Q4KPlain>(ps, &o.p, o.stages, smem, link);
            } else {
                if (tid < (uint32_t)Q6KPlain::THREADS) run_stages<Q6K, Q6KPlain>(ps, &o.p, o.stages, smem, link);
            }
            prev_slots = o.slots;
            prev_stages = o.stages;
        } else if (i == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
        } else if (tid == 0) {
            // no part in this operator, but the count is a sum over blocks: a block may only arrive for an
            // operator once it has seen every block finish the one before
            bool there = false;
            for (uint32_t k = 0; k < CHAIN_SPIN_LIMIT && !there; ++k) {
                there = ld_acquire_u32(link.arrivals) >= link.target;
                if (!there) __nanosleep(64);
            }
            if (!there) atomicExch(o.p.status, 1u);
        }
    }
    // the last block to leave puts the counters back to zero for the next launch
    __syncthreads();
    if (tid == 0 && c.count > 1) {
        __threadfence();
        if (atomicAdd(c.arrivals + 1, 1u) == gridDim.x - 1) {
            c.arrivals[0] = 0;
            c.arrivals[1] = 0;
            __threadfence();
        }
    }
}

}  // namespace i8

bool chain_configure() {
    return cudaFuncSetAttribute(i8::chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)i8::kSmemMax) == cudaSuccess;
}

// Whether a job can be a link of a chain: one token, a weight stream that may start early, no fused push.
bool chain_supported(const FastJob &job) {
    if (job.tokens != 1 || job.serial || job.push.ranks || job.norm_weight || job.add0) return false;
    i8::Params p;
    i8::Plan plan;
    return (q4k_i8_fill(job, p, plan, false) || q6k_i8_fill(job, p, plan, false)) && plan.nt == 1;
}

// Launches jobs[0..n) (2 <= n <= kChainMax, each chain_supported) in order as one kernel. arrivals: two words, zero.
int launch_chain(cudaStream_t s, const FastJob *jobs, uint32_t n, uint32_t *arrivals, int sm_count) {
    static thread_local i8::ChainParams c;
    if (n < 2 || n > (uint32_t)kChainMax) return 0;
    c.count = n;
    c.arrivals = arrivals;
    size_t smem = 0;
    for (uint32_t i = 0; i < n; ++i) {
        i8::ChainOp &o = c.op[i];
        i8::Plan plan;
        if (q4k_i8_fill(jobs[i], o.p, plan, true)) {
            o.kind = i8::CHAIN_Q4K;
            o.slots = i8::Q4KPlain::SLOTS;
        } else if (q6k_i8_fill(jobs[i], o.p, plan, true)) {
            o.kind = i8::CHAIN_Q6K;
            o.slots = i8::Q6KPlain::SLOTS;
        } else {
            return 0;
        }
        if (plan.nt != 1 || plan.grid > (uint32_t)sm_count) return 0;
        o.stages = (uint32_t)plan.stages;
        o.grid = plan.grid;
        smem = plan.smem > smem ? plan.smem : smem;
    }
    // cooperative: every block resident at once, or the launch fails; it may still start under the tail of the kernel before it
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)sm_count);
    cfg.blockDim = dim3(i8::kChainThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, i8::chain_kernel, c);
    return 1;
}

}  // namespace nu
