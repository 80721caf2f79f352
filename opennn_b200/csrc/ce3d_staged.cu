// CrossEntropyError3d in ONE pass over HBM (opennn/cross_entropy_error_3d.cpp:78-136 error, :154-247 output gradients):
// every logit is read from global memory once and every gradient written once.
//
// A row of V logits (128 KB at V = 32000) does not fit in registers, and a second sweep through global memory costs a
// third of the kernel's traffic, so the row is staged in shared memory.  One persistent CTA per SM walks token rows.
// Shared memory is a ring of 8 KiB slots; a producer thread streams the rows' chunks into free slots with bulk copies
// (cp.async.bulk, completion counted on one mbarrier per slot) and runs ahead into the following rows as far as the
// ring allows, so the loads of the next row are in flight while this row is being reduced and written back.  The 512
// consumer threads take maximum, sum of exponentials and arg-max of a row chunk by chunk as the chunks land, combine
// them once per row, turn the staged logits into gradients IN PLACE in shared memory and hand each chunk back to the
// producer thread, which writes it to global memory with a bulk store and reuses the slot when the store has read it.
// Rows whose target is padding need no logits at all: the consumers write their zeros directly.
//
// Every mbarrier wait is bounded; a wait that runs out records a status word (ce3d_staged_read_status), the CTA
// waits (bounded again) for its bulk copies in flight and returns.
#include <float.h>

#include "common.cuh"
#include "launch_counter.h"
#include "rowwise_internal.h"
#include "tcgen05.cuh"

namespace onn
{

namespace
{

constexpr int kChunkFloats = 2048;                    // 8 KiB per bulk copy; one float4 per consumer thread
constexpr int kChunkBytes = kChunkFloats * 4;
constexpr int kConsumers = 512;
constexpr int kConsumerWarps = kConsumers / 32;
constexpr int kThreads = kConsumers + 32;             // + the producer warp (one thread of it works)
constexpr int kSlots = 27;                            // 27 x 8 KiB = 216 KiB of the 227 KiB a CTA may use
constexpr int kMinStagedV = 4096;                     // shorter rows: one small CTA per row is as good and simpler

struct Control
{
    unsigned long long full[kSlots];               // producer -> consumers: the chunk has landed
    unsigned long long done[kSlots];               // consumers -> producer: the chunk holds gradients, store it
    float part_max[2][kConsumerWarps];
    float part_sum[2][kConsumerWarps];
    int part_arg[2][kConsumerWarps];
    int consumer_abort;                               // written by consumers only, read by them after a barrier
    int producer_abort;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(dst), "r"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" :: "n"(kConsumers) : "memory"); }

__device__ __forceinline__ bool row_is_active(const float* __restrict__ targets, long long r, int V)
{
    const long long t = token_index(__ldg(targets + r));
    return t > 0 && t < V;
}

__global__ void __launch_bounds__(kThreads, 1)
ce3d_staged_kernel(float* __restrict__ logits, const float* __restrict__ targets, const float* __restrict__ active_count,
                   float* __restrict__ row_scratch, long long rows, int V, int inputs_are_probabilities)
{
    extern __shared__ __align__(128) unsigned char shared_bytes[];
    float* ring = reinterpret_cast<float*>(shared_bytes);
    Control* control = reinterpret_cast<Control*>(shared_bytes + (size_t)kSlots * kChunkBytes);
    const int chunks = (V + kChunkFloats - 1) / kChunkFloats;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < kSlots; s++)
        {
            tc::mbar_init(tc::smem_u32(control->full + s), 1);
            tc::mbar_init(tc::smem_u32(control->done + s), kConsumerWarps);
        }
        control->consumer_abort = 0;
        control->producer_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if(threadIdx.x >= kConsumers)
    {
        // ---- producer: loads into free slots, stores of finished chunks, in ring order ----
        if(threadIdx.x != kConsumers) return;
        const long long step = gridDim.x;
        auto next_staged = [&](long long r) { while(r < rows && !row_is_active(targets, r, V)) r += step; return r; };
        // chunks are numbered in ring order; a chunk's slot is its number modulo the ring size and its barrier phase the
        // parity of the ring's laps, both kept incrementally
        unsigned int loaded = 0, stored = 0, freed = 0;
        long long load_row = next_staged(blockIdx.x), store_row = load_row;
        int load_chunk = 0, store_chunk = 0, load_slot = 0, store_slot = 0;
        uint32_t store_phase = 0;
        bool failed = false;
        while(true)
        {
            while(load_row < rows && loaded - freed < (unsigned int)kSlots)
            {
                const int first = load_chunk * kChunkFloats;
                const uint32_t bytes = (uint32_t)min(kChunkFloats, V - first) * 4u;
                const uint32_t bar = tc::smem_u32(control->full + load_slot);
                tc::mbar_arrive_expect_tx(bar, bytes);
                bulk_load(tc::smem_u32(ring + (size_t)load_slot * kChunkFloats), logits + load_row * (long long)V + first, bytes, bar);
                loaded++;
                if(++load_slot == kSlots) load_slot = 0;
                if(++load_chunk == chunks) { load_chunk = 0; load_row = next_staged(load_row + step); }
            }
            if(stored == loaded)
            {
                if(load_row >= rows) break;
                tc::bulk_wait_read_0();                 // every slot holds a store that has not been read out yet
                freed = stored;
                continue;
            }
            if(!tc::mbar_wait(tc::smem_u32(control->done + store_slot), store_phase, &control->producer_abort, 0xCE01u))
            {
                failed = true;
                break;
            }
            const int first = store_chunk * kChunkFloats;
            const uint32_t bytes = (uint32_t)min(kChunkFloats, V - first) * 4u;
            bulk_store(logits + store_row * (long long)V + first, tc::smem_u32(ring + (size_t)store_slot * kChunkFloats), bytes);
            tc::bulk_commit();
            stored++;
            if(++store_slot == kSlots) { store_slot = 0; store_phase ^= 1u; }
            if(++store_chunk == chunks) { store_chunk = 0; store_row = next_staged(store_row + step); }
            tc::bulk_wait_read_1();                     // all stores but the newest have left shared memory
            freed = stored - 1;
        }
        if(failed)
        {
            // loads still in flight must land before this CTA's shared memory is given up
            int ignore = 0;
            for(unsigned int n = stored; n != loaded; n++)
            {
                tc::mbar_wait(tc::smem_u32(control->full + store_slot), store_phase, &ignore, 0xCE02u);
                if(++store_slot == kSlots) { store_slot = 0; store_phase ^= 1u; }
            }
        }
        tc::bulk_wait_all();
        return;
    }

    // ---- consumers ----
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float count = active_count[0];
    const float scale = count > 0.f ? 1.0f / count : 0.f;
    int row_slot = 0;                                   // ring slot and barrier phase of the row's first chunk
    uint32_t row_phase = 0;
    int flip = 0;
    for(long long r = blockIdx.x; r < rows; r += gridDim.x)
    {
        float* row = logits + r * (long long)V;
        const long long target = token_index(__ldg(targets + r));
        if(!(target > 0 && target < V))
        {
            // nothing of this row is needed: the gradient is zero and it adds nothing to the loss
            for(int i = tid * 4; i < V; i += kConsumers * 4) st4_stream(row + i, make_float4(0.f, 0.f, 0.f, 0.f));
            if(tid == 0) { row_scratch[r] = 0.f; row_scratch[rows + r] = 0.f; }
            continue;
        }

        // sweep 1, from shared memory as the chunks land: maximum, sum of exponentials, first arg-max
        float m = -INFINITY, s = 0.f;
        int arg = 0x7fffffff;
        int slot = row_slot;
        uint32_t phase = row_phase;
        for(int c = 0; c < chunks; c++)
        {
            if(!tc::mbar_wait(tc::smem_u32(control->full + slot), phase, &control->consumer_abort, 0xCE03u)) break;
            const int i = c * kChunkFloats + tid * 4;
            if(i < V)
            {
                const float4 x = ld4(ring + (size_t)slot * kChunkFloats + tid * 4);
                float nm = m;
                if(x.x > nm) { nm = x.x; arg = i; }
                if(x.y > nm) { nm = x.y; arg = i + 1; }
                if(x.z > nm) { nm = x.z; arg = i + 2; }
                if(x.w > nm) { nm = x.w; arg = i + 3; }
                if(nm > m) { s *= __expf(m - nm); m = nm; }
                if(m > -INFINITY) s += (__expf(x.x - m) + __expf(x.y - m)) + (__expf(x.z - m) + __expf(x.w - m));
            }
            if(++slot == kSlots) { slot = 0; phase ^= 1u; }
        }
#pragma unroll
        for(int offset = 16; offset > 0; offset >>= 1)
        {
            const float om = __shfl_xor_sync(0xffffffffu, m, offset);
            const float os = __shfl_xor_sync(0xffffffffu, s, offset);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, offset);
            const float nm = fmaxf(m, om);
            const float a = (m == -INFINITY) ? 0.f : s * __expf(m - nm);
            const float b = (om == -INFINITY) ? 0.f : os * __expf(om - nm);
            if(om > m || (om == m && oa < arg)) arg = oa;
            m = nm; s = a + b;
        }
        if(lane == 0) { control->part_max[flip][warp] = m; control->part_sum[flip][warp] = s; control->part_arg[flip][warp] = arg; }
        consumer_barrier();
        if(*(volatile int*)&control->consumer_abort) break;      // the same for every consumer: set only before the barrier
        m = control->part_max[flip][0]; s = control->part_sum[flip][0]; arg = control->part_arg[flip][0];
#pragma unroll
        for(int w = 1; w < kConsumerWarps; w++)
        {
            const float om = control->part_max[flip][w], os = control->part_sum[flip][w];
            const int oa = control->part_arg[flip][w];
            const float nm = fmaxf(m, om);
            const float a = (m == -INFINITY) ? 0.f : s * __expf(m - nm);
            const float b = (om == -INFINITY) ? 0.f : os * __expf(om - nm);
            if(om > m || (om == m && oa < arg)) arg = oa;      // ties: the first maximum, as the reference's scan
            m = nm; s = a + b;
        }
        const float shift = inputs_are_probabilities ? 0.f : m;
        const float inv = inputs_are_probabilities ? 1.0f : (s > 0.f ? 1.0f / s : 0.f);
        const int t = (int)target;

        // sweep 2, in place in shared memory: the gradient (p - onehot) / active; each finished chunk goes to the producer
        slot = row_slot;
        for(int c = 0; c < chunks; c++)
        {
            const int i = c * kChunkFloats + tid * 4;
            if(i < V)
            {
                float* at = ring + (size_t)slot * kChunkFloats + tid * 4;
                float4 x = ld4(at);
                const float p0 = inputs_are_probabilities ? x.x : __expf(x.x - shift) * inv;
                const float p1 = inputs_are_probabilities ? x.y : __expf(x.y - shift) * inv;
                const float p2 = inputs_are_probabilities ? x.z : __expf(x.z - shift) * inv;
                const float p3 = inputs_are_probabilities ? x.w : __expf(x.w - shift) * inv;
                if((unsigned)(t - i) < 4u)
                {
                    const float p = t == i ? p0 : t == i + 1 ? p1 : t == i + 2 ? p2 : p3;
                    row_scratch[r] = -logf(p + FLT_EPSILON);
                    row_scratch[rows + r] = (arg == t) ? 1.f : 0.f;
                }
                x.x = (p0 - (i == t ? 1.0f : 0.0f)) * scale;
                x.y = (p1 - (i + 1 == t ? 1.0f : 0.0f)) * scale;
                x.z = (p2 - (i + 2 == t ? 1.0f : 0.0f)) * scale;
                x.w = (p3 - (i + 3 == t ? 1.0f : 0.0f)) * scale;
                st4(at, x);
            }
            tc::fence_async_shared();                    // these writes, then the bulk store's reads
            __syncwarp();
            if(lane == 0) tc::mbar_arrive(tc::smem_u32(control->done + slot));
            if(++slot == kSlots) { slot = 0; row_phase ^= 1u; }
        }
        row_slot = slot;
        flip ^= 1;
    }
}

PerDeviceBytes g_staged_smem;

}  // namespace

bool ce3d_staged_takes(const float* logits, const float* probabilities_out, long long rows, long long V)
{
    if(probabilities_out || rows <= 0) return false;
    if(V < kMinStagedV || (V & 3) != 0 || !host_aligned16(logits)) return false;
    return (V + kChunkFloats - 1) / kChunkFloats <= kSlots;
}

int ce3d_staged_launch(float* logits, const float* targets, const float* active_count, float* row_scratch,
                       long long rows, int V, int inputs_are_probabilities, cudaStream_t stream)
{
    // the ring holds the row being worked on plus as many chunks of the following rows as fit
    const size_t shared = (size_t)kSlots * kChunkBytes + sizeof(Control);
    if(!ensure_dynamic_smem(ce3d_staged_kernel, g_staged_smem, shared)) return ONN_ERR_CUDA;
    const int grid = (int)(rows < sm_limit() ? rows : sm_limit());
    ce3d_staged_kernel<<<grid, kThreads, shared, stream>>>(logits, targets, active_count, row_scratch, rows, V,
                                                           inputs_are_probabilities);
    count_launch();
    return launch_status();
}

const unsigned int* ce3d_staged_status_word() { return tc::status_word_address(); }

int ce3d_staged_read_status()
{
    unsigned int status = 0;
    if(tc::read_and_clear_status(&status) != 0) return ONN_ERR_CUDA;
    return status == 0 ? ONN_OK : ONN_ERR_DEVICE_TIMEOUT;
}

}  // namespace onn
