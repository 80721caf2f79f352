// CrossEntropyError3d in ONE pass over HBM (opennn/cross_entropy_error_3d.cpp:78-136 error, :154-247 output gradients):
// every logit is read from global memory once and every gradient written once.
//
// One persistent CTA per SM walks token rows and holds the row it works on in REGISTERS: 992 consumer threads, one
// float4 of every 3968-float chunk each, up to 9 chunks (V <= 35712; 128 KB at V = 32000, half the register file).
// The logits get there through a ring of 13 shared-memory slots: a producer thread streams the chunks of this CTA's
// rows into free slots with bulk copies (cp.async.bulk, completion counted on one mbarrier per slot) and a slot goes
// back to it as soon as every consumer warp has taken its part of the chunk into registers.  The ring therefore
// holds what is still to come, about a row and a half, so the loads of the next row are in flight while this row is
// being worked on; shared memory is transit only and nothing is ever written back to it.  Per row the consumers
//   A  take the chunks into registers as they land, with the row maximum and the first arg-max;
//   B  turn them into e = exp(x - max) in place, with the sum;
//   C  write the gradient (e / sum - onehot) / active to global memory with 128-bit streaming stores.
// One exponential per logit; two CTA-wide combines per row.
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

constexpr int kConsumers = 992;                       // 31 warps + the producer's warp = the 1024 threads a CTA may have
constexpr int kConsumerWarps = kConsumers / 32;
constexpr int kChunkFloats = kConsumers * 4;          // 15.5 KiB per bulk copy; one float4 per consumer thread
constexpr int kChunkBytes = kChunkFloats * 4;
constexpr int kThreads = kConsumers + 32;             // + the producer warp (one thread of it works)
constexpr int kSlots = 13;                            // 13 x 15.5 KiB = 201.5 KiB of the 227 KiB a CTA may use
constexpr int kMaxChunks = 9;                         // chunks of a row a consumer thread can hold: 36 registers
constexpr int kMinStagedV = 4096;                     // shorter rows: one small CTA per row is as good and simpler
constexpr float kLog2e = 1.4426950408889634f;

struct Control
{
    unsigned long long full[kSlots];                  // producer -> consumers: the chunk has landed
    unsigned long long done[kSlots];                  // consumers -> producer: every warp has taken its part of the chunk
    float part_a[2][kConsumerWarps];                  // per-warp maxima, then per-warp sums
    int part_arg[2][kConsumerWarps];
    int consumer_abort;                               // written by consumers only, read by them after a barrier
    int producer_abort;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" :: "n"(kConsumers) : "memory"); }

__device__ __forceinline__ float exp2_fast(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed fp32: one instruction for two elements (fma.rn.f32x2 / mul.f32x2 / add.f32x2 of sm_100).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c)
{
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

__device__ __forceinline__ float2 mul2(float2 a, float2 b)
{
    unsigned long long ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

__device__ __forceinline__ float2 add2(float2 a, float2 b)
{
    unsigned long long ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

__device__ __forceinline__ bool row_is_active(const float* __restrict__ targets, long long r, int V)
{
    const long long t = token_index(__ldg(targets + r));
    return t > 0 && t < V;
}

template <int CHUNKS>                                 // the row's chunk count: the size of a consumer thread's register array
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
        // ---- producer: streams the chunks of this CTA's active rows into the ring, in order ----
        if(threadIdx.x != kConsumers) return;
        const long long step = gridDim.x;
        auto next_staged = [&](long long r) { while(r < rows && !row_is_active(targets, r, V)) r += step; return r; };
        // chunks are numbered in ring order: chunk n lives in slot n % kSlots, and a slot may be refilled when the
        // consumers have released the chunk that was in it one lap of the ring earlier
        unsigned int loaded = 0;
        long long load_row = next_staged(blockIdx.x);
        int load_chunk = 0, slot = 0;
        bool failed = false;
        while(load_row < rows)
        {
            // chunk n refills its slot after the release of chunk n - kSlots: the slot's release number n / kSlots - 1
            if(loaded >= (unsigned int)kSlots &&
               !tc::mbar_wait(tc::smem_u32(control->done + slot), (loaded / kSlots - 1u) & 1u, &control->producer_abort, 0xCE01u))
            {
                failed = true;
                break;
            }
            const int first = load_chunk * kChunkFloats;
            const uint32_t bytes = (uint32_t)min(kChunkFloats, V - first) * 4u;
            const uint32_t bar = tc::smem_u32(control->full + slot);
            tc::mbar_arrive_expect_tx(bar, bytes);
            bulk_load(tc::smem_u32(ring + (size_t)slot * kChunkFloats), logits + load_row * (long long)V + first, bytes, bar);
            loaded++;
            if(++slot == kSlots) slot = 0;
            if(++load_chunk == chunks) { load_chunk = 0; load_row = next_staged(load_row + step); }
        }
        if(failed)
        {
            // loads still in flight must land before this CTA's shared memory is given up: the last lap of the ring
            int ignore = 0;
            const unsigned int in_ring = loaded < (unsigned int)kSlots ? loaded : (unsigned int)kSlots;
            for(unsigned int back = 1; back <= in_ring; back++)
            {
                const unsigned int n = loaded - back;
                tc::mbar_wait(tc::smem_u32(control->full + (int)(n % kSlots)), (n / kSlots) & 1u, &ignore, 0xCE02u);
            }
        }
        return;
    }

    // ---- consumers ----
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float count = active_count[0];
    const float scale = count > 0.f ? 1.0f / count : 0.f;
    const float* mine = ring + tid * 4;                 // this thread's float4 of slot 0; slot s is s * kChunkFloats further
    int slot = 0;                                       // ring slot and barrier phase of the next chunk to take
    uint32_t phase = 0;
    int flip = 0;
    long long target = blockIdx.x < rows ? token_index(__ldg(targets + blockIdx.x)) : 0;
    for(long long r = blockIdx.x; r < rows; r += gridDim.x)
    {
        float* row = logits + r * (long long)V;
        const int t = (target > 0 && target < V) ? (int)target : -1;
        // the next row's target is fetched now: nothing of that row can start without it
        const long long r_next = r + gridDim.x;
        if(r_next < rows) target = token_index(__ldg(targets + r_next));
        if(t < 0)
        {
            // nothing of this row is needed: the gradient is zero and it adds nothing to the loss
            for(int i = tid * 4; i < V; i += kConsumers * 4) st4_stream(row + i, make_float4(0.f, 0.f, 0.f, 0.f));
            if(tid == 0) { row_scratch[r] = 0.f; row_scratch[rows + r] = 0.f; }
            continue;
        }

        // sweep A, as the chunks land: into registers, with the maximum and first arg-max of this thread's elements;
        // a chunk every warp has taken goes back to the producer at once
        float4 x[CHUNKS];
        float m = -INFINITY;
        int arg = 0x7fffffff;
        bool landed = true;
#pragma unroll
        for(int c = 0; c < CHUNKS; c++)
        {
            if(!landed) break;
            // the chunk is usually there already; if not, one lane waits (bounded) and the others then look once more
            if(!tc::mbar_try_wait(tc::smem_u32(control->full + slot), phase))
            {
                if(lane == 0) landed = tc::mbar_wait(tc::smem_u32(control->full + slot), phase, &control->consumer_abort, 0xCE03u);
                landed = __shfl_sync(0xffffffffu, landed, 0);
                if(!landed) break;
                tc::mbar_try_wait(tc::smem_u32(control->full + slot), phase);
            }
            const int i = c * kChunkFloats + tid * 4;
            x[c] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            if(c < CHUNKS - 1 || i < V)                // only the row's last chunk can be ragged
            {
                x[c] = ld4(mine + (size_t)slot * kChunkFloats);
                if(x[c].x > m) { m = x[c].x; arg = i; }
                if(x[c].y > m) { m = x[c].y; arg = i + 1; }
                if(x[c].z > m) { m = x[c].z; arg = i + 2; }
                if(x[c].w > m) { m = x[c].w; arg = i + 3; }
            }
            __syncwarp();
            if(lane == 0) tc::mbar_arrive(tc::smem_u32(control->done + slot));
            if(++slot == kSlots) { slot = 0; phase ^= 1u; }
        }
#pragma unroll
        for(int offset = 16; offset > 0; offset >>= 1)
        {
            const float om = __shfl_xor_sync(0xffffffffu, m, offset);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, offset);
            if(om > m || (om == m && oa < arg)) { m = om; arg = oa; }      // ties: the first maximum, as the reference's scan
        }
        if(lane == 0) { control->part_a[flip][warp] = m; control->part_arg[flip][warp] = arg; }
        consumer_barrier();
        if(*(volatile int*)&control->consumer_abort) break;      // the same for every consumer: set only before the barrier
        m = lane < kConsumerWarps ? control->part_a[flip][lane] : -INFINITY;
        arg = lane < kConsumerWarps ? control->part_arg[flip][lane] : 0x7fffffff;
#pragma unroll
        for(int offset = 16; offset > 0; offset >>= 1)
        {
            const float om = __shfl_xor_sync(0xffffffffu, m, offset);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, offset);
            if(om > m || (om == m && oa < arg)) { m = om; arg = oa; }
        }
        flip ^= 1;

        // sweep B: e = exp(x - max) in place, and its sum (probabilities in: they are used as they are); two elements per
        // multiply-add and per add (the packed fp32 instructions of this architecture)
        float inv = 1.0f;
        if(!inputs_are_probabilities)
        {
            const float shift = m > -INFINITY ? m * kLog2e : 0.f;
            const float2 scale2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(-shift, -shift);
            float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
            for(int c = 0; c < CHUNKS; c++)
            {
                const float2 lo = fma2(make_float2(x[c].x, x[c].y), scale2, shift2), hi = fma2(make_float2(x[c].z, x[c].w), scale2, shift2);
                x[c].x = exp2_fast(lo.x); x[c].y = exp2_fast(lo.y); x[c].z = exp2_fast(hi.x); x[c].w = exp2_fast(hi.y);
                sum2 = add2(sum2, add2(make_float2(x[c].x, x[c].y), make_float2(x[c].z, x[c].w)));   // past the row's end: exp(-inf) = 0
            }
            float s = warp_sum(sum2.x + sum2.y);
            if(lane == 0) control->part_a[flip][warp] = s;
            consumer_barrier();
            s = warp_sum(lane < kConsumerWarps ? control->part_a[flip][lane] : 0.f);
            flip ^= 1;
            inv = s > 0.f ? 1.0f / s : 0.f;
        }
        const float pick = inv * scale;                  // e -> gradient of an off-target logit
        const float2 pick2 = make_float2(pick, pick);

        // sweep C, from registers to global memory: e * pick everywhere, then the one thread that holds the target
        // element writes that element again with the one-hot term (same thread, same address: the later store stays)
        float* out = row + tid * 4;
#pragma unroll
        for(int c = 0; c < CHUNKS; c++)
        {
            if(c < CHUNKS - 1 || c * kChunkFloats + tid * 4 < V)
            {
                const float2 lo = mul2(make_float2(x[c].x, x[c].y), pick2), hi = mul2(make_float2(x[c].z, x[c].w), pick2);
                st4_stream(out + c * kChunkFloats, make_float4(lo.x, lo.y, hi.x, hi.y));
            }
        }
        const int mine_first = t - tid * 4;              // the target is mine if this is c * kChunkFloats + k with 0 <= k < 4
        const int owner_chunk = mine_first / kChunkFloats, k = mine_first - owner_chunk * kChunkFloats;
        if(mine_first >= 0 && k < 4)
        {
            float e = 0.f;
#pragma unroll
            for(int c = 0; c < CHUNKS; c++)
                if(c == owner_chunk) e = k == 0 ? x[c].x : k == 1 ? x[c].y : k == 2 ? x[c].z : x[c].w;
            row_scratch[r] = -logf(e * inv + FLT_EPSILON);
            row_scratch[rows + r] = (arg == t) ? 1.f : 0.f;
            row[t] = fmaf(e, pick, -scale);
        }
    }
}

}  // namespace

bool ce3d_staged_takes(const float* logits, const float* probabilities_out, long long rows, long long V)
{
    if(probabilities_out || rows <= 0) return false;
    if(V < kMinStagedV || (V & 3) != 0 || !host_aligned16(logits)) return false;
    return (V + kChunkFloats - 1) / kChunkFloats <= kMaxChunks;
}

namespace
{
template <int CHUNKS>
int launch_staged(float* logits, const float* targets, const float* active_count, float* row_scratch,
                  long long rows, int V, int inputs_are_probabilities, cudaStream_t stream)
{
    static PerDeviceBytes configured;                      // per instantiation and per device
    const size_t shared = (size_t)kSlots * kChunkBytes + sizeof(Control);
    if(!ensure_dynamic_smem(ce3d_staged_kernel<CHUNKS>, configured, shared)) return ONN_ERR_CUDA;
    const int grid = (int)(rows < sm_limit() ? rows : sm_limit());
    ce3d_staged_kernel<CHUNKS><<<grid, kThreads, shared, stream>>>(logits, targets, active_count, row_scratch, rows, V,
                                                                   inputs_are_probabilities);
    count_launch();
    return launch_status();
}
}  // namespace

int ce3d_staged_launch(float* logits, const float* targets, const float* active_count, float* row_scratch,
                       long long rows, int V, int inputs_are_probabilities, cudaStream_t stream)
{
    // the register array of a consumer thread and its unrolled sweeps are sized by the row's chunk count
    switch((V + kChunkFloats - 1) / kChunkFloats)
    {
#define ONN_STAGED(N) case N: return launch_staged<N>(logits, targets, active_count, row_scratch, rows, V, inputs_are_probabilities, stream)
        ONN_STAGED(2); ONN_STAGED(3); ONN_STAGED(4); ONN_STAGED(5); ONN_STAGED(6); ONN_STAGED(7); ONN_STAGED(8); ONN_STAGED(9);
#undef ONN_STAGED
        default: return ONN_ERR_UNSUPPORTED;
    }
}

const unsigned int* ce3d_staged_status_word() { return tc::status_word_address(); }

int ce3d_staged_read_status()
{
    unsigned int status = 0;
    if(tc::read_and_clear_status(&status) != 0) return ONN_ERR_CUDA;
    return status == 0 ? ONN_OK : ONN_ERR_DEVICE_TIMEOUT;
}

}  // namespace onn
