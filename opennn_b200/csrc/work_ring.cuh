// Work items of a persistent one-CTA kernel, handed from one scheduling thread to the kernel's other roles.
//
// The kernels built on tcgen05.cuh split a CTA into roles (copy producer, MMA issuer, arithmetic warps) that all walk the
// same sequence of work items.  With a fixed share per CTA (item = blockIdx.x + turn * gridDim.x) every role can compute
// the sequence itself; when the items come from a global counter (common.cuh: next_work_counter) one thread asks the
// counter and the others must be told.  The ring below does that: kWorkRing slots in shared memory, a "full" barrier per
// slot that the scheduler completes after writing the item number, an "empty" barrier that every reading role arrives on
// once it has the number in a register.  Item kNoWork ends the sequence.  All waits are bounded like every other wait of
// these kernels.
#pragma once
#include "tcgen05.cuh"

namespace onn
{
namespace tc
{

constexpr int kWorkRing = 4;
constexpr uint32_t kNoWork = 0xffffffffu;

struct WorkRing
{
    uint64_t full[kWorkRing];
    uint64_t empty[kWorkRing];
    uint32_t item[kWorkRing];
    uint32_t reserved[2];
};
static_assert(sizeof(WorkRing) == 88, "shared-memory budgets of the kernels count on this");

// one thread, together with the kernel's other barrier initialisations (before their fence); `readers` = reading roles
__device__ __forceinline__ void work_ring_init(WorkRing* ring, uint32_t readers)
{
    for(int r = 0; r < kWorkRing; r++) { mbar_init(smem_u32(ring->full + r), 1); mbar_init(smem_u32(ring->empty + r), readers); }
}

// The work-item source of one launch: a counter, or (null) the fixed share of this CTA.
struct WorkSource
{
    unsigned int* counter;
    uint32_t total;                                          // work items of the launch
    uint32_t schedulers;                                     // scheduling threads of the launch (one per CTA, or per CTA pair)

    // scheduler: the number of the next item, kNoWork past the end; it stops asking at the first kNoWork.  With a counter
    // this is one atomic round trip: ask early, use late.  Every scheduler asks exactly once past the end, so the launch
    // asks total + schedulers times in all, and the counter -- an increment that wraps at that number -- is back at zero
    // when the last of them has asked: nothing to clear, no second counter, and the replay of a captured launch finds
    // it as the capture did.
    __device__ __forceinline__ uint32_t fetch(uint32_t turn, uint32_t share_first, uint32_t share_stride) const
    {
        const uint32_t w = counter ? atomicInc(counter, total + schedulers - 1u) : share_first + turn * share_stride;
        return w < total ? w : kNoWork;
    }
};

// scheduler: item number `item` becomes turn `turn` of every reading role.  The callers below skip the ring altogether
// when the launch has no counter: every role can then compute its items itself, as a kernel without a ring would.
__device__ __forceinline__ bool work_ring_publish(WorkRing* ring, uint32_t turn, uint32_t item, volatile int* abort_flag, unsigned int site)
{
    const uint32_t slot = turn % kWorkRing, parity = (turn / kWorkRing) & 1u;
    if(!mbar_wait(smem_u32(ring->empty + slot), parity ^ 1u, abort_flag, site)) return false;
    *reinterpret_cast<volatile uint32_t*>(ring->item + slot) = item;
    mbar_arrive(smem_u32(ring->full + slot));
    return true;
}

// reading role (one thread of it): the item of turn `turn`, without handing the slot back -- a role that wants to know
// its NEXT item early looks at turn + 1 this way and takes it when its turn comes.  kNoWork also when the wait gave up.
__device__ __forceinline__ uint32_t work_ring_peek(WorkRing* ring, uint32_t turn, volatile int* abort_flag, unsigned int site)
{
    const uint32_t slot = turn % kWorkRing, parity = (turn / kWorkRing) & 1u;
    if(!mbar_wait(smem_u32(ring->full + slot), parity, abort_flag, site)) return kNoWork;
    return *reinterpret_cast<volatile uint32_t*>(ring->item + slot);
}

// hands the slot of turn `turn` back; `item` is what the role read there -- the slot goes back once that number is in a
// register (the branch needs it).  The arrival publishes nothing, so it is relaxed: a release would make the MMA issuer
// wait for the MMAs it has in flight.
__device__ __forceinline__ void work_ring_release(WorkRing* ring, uint32_t turn, uint32_t item)
{
    if(item != kNoWork - 1u)
        asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" :: "r"(smem_u32(ring->empty + (turn % kWorkRing))) : "memory");
}

__device__ __forceinline__ uint32_t work_ring_take(WorkRing* ring, uint32_t turn, volatile int* abort_flag, unsigned int site)
{
    const uint32_t item = work_ring_peek(ring, turn, abort_flag, site);
    work_ring_release(ring, turn, item);
    return item;
}

// What a role of a one-CTA kernel uses: the ring when the launch hands its items out by counter, plain arithmetic on the
// CTA's fixed share when it does not.
struct WorkView
{
    WorkRing* ring;
    bool by_counter;
    uint32_t total;

    __device__ __forceinline__ uint32_t fixed(uint32_t turn) const
    {
        const uint32_t w = blockIdx.x + turn * gridDim.x;
        return w < total ? w : kNoWork;
    }
    __device__ __forceinline__ bool publish(uint32_t turn, uint32_t item, volatile int* abort_flag, unsigned int site) const
    {
        return by_counter ? work_ring_publish(ring, turn, item, abort_flag, site) : true;
    }
    __device__ __forceinline__ uint32_t peek(uint32_t turn, volatile int* abort_flag, unsigned int site) const
    {
        return by_counter ? work_ring_peek(ring, turn, abort_flag, site) : fixed(turn);
    }
    __device__ __forceinline__ void release(uint32_t turn, uint32_t item) const
    {
        if(by_counter) work_ring_release(ring, turn, item);
    }
    __device__ __forceinline__ uint32_t take(uint32_t turn, volatile int* abort_flag, unsigned int site) const
    {
        return by_counter ? work_ring_take(ring, turn, abort_flag, site) : fixed(turn);
    }
    // the same for a whole warp (all lanes call, all lanes get the number): lane 0 asks the ring and hands the answer
    // round; with fixed shares every lane computes it and nothing is exchanged
    __device__ __forceinline__ uint32_t warp_peek(uint32_t turn, int lane, volatile int* abort_flag, unsigned int site) const
    {
        if(!by_counter) return fixed(turn);
        uint32_t w = 0;
        if(lane == 0) w = work_ring_peek(ring, turn, abort_flag, site);
        return __shfl_sync(0xffffffffu, w, 0);
    }
    __device__ __forceinline__ void warp_release(uint32_t turn, uint32_t item, int lane) const
    {
        if(by_counter && lane == 0) work_ring_release(ring, turn, item);
    }
    __device__ __forceinline__ uint32_t warp_take(uint32_t turn, int lane, volatile int* abort_flag, unsigned int site) const
    {
        const uint32_t w = warp_peek(turn, lane, abort_flag, site);
        warp_release(turn, w, lane);
        return w;
    }
};

}  // namespace tc
}  // namespace onn
