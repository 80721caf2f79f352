// tcgen05 GEMM for sm_100a: fp32 storage consumed as tf32 (kind::tf32), fp32 accumulation
// in tensor memory.
//
// One persistent CTA per SM walks a static list of 128 x BN output tiles.  Six warps:
//   warp 0      TMA producer: cp.async.bulk.tensor (4-D maps, 128-byte swizzle, zero fill
//               out of bounds) into a ring of shared-memory stages, one mbarrier each way;
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128 x BN x 8 from shared-memory
//               descriptors; owns the TMEM allocation (two accumulator buffers so the
//               epilogue of tile i overlaps the main loop of tile i+1);
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM lanes = 32
//               output rows), alpha / bias / ReLU, stage the 32 x 32 block in shared memory
//               (128-byte swizzle) and hand it to a TMA store -- or a TMA reduce-add for
//               accumulation and split-K -- so global writes are whole lines and clipped at the
//               matrix edge by the copy engine.  What the epilogue reads from global memory (bias
//               values, the ReLU mask as one bit per element) is fetched once per tile BEFORE the
//               wait for the accumulator, so its latency passes behind the MMAs; a float ReLU-mask
//               operand and column sums of the output are applied to the staged block.
//
// Operand layouts (BK = 32 floats = 128 bytes = one swizzle row, UMMA K = 8):
//   K-major  (reduction dimension contiguous in memory): one box [rows][32 floats];
//            canonical K-major SWIZZLE_128B layout, 8-row groups 1024 bytes apart (SBO);
//            the K step inside a stage advances the descriptor start address by 32 bytes.
//   MN-major (M or N contiguous in memory): one box [32 k-rows][32 floats] per 32 columns,
//            written with the 128-byte swizzle whose atom is 32 bytes (the only MN-major
//            layout tf32 operands have: SWIZZLE_128B_BASE32B, pattern period 4 rows); boxes
//            4096 bytes apart (LBO), 4-row k-groups 512 bytes apart (SBO); the K step (8
//            rows) advances the start address by 1024 bytes.
//
// The tensor maps carry the TFLOAT32 data type: the TMA unit then rounds every fp32 element
// to the nearest tf32 value (ties to even) on its way into shared memory, so the tensor
// cores -- which ignore the low 13 mantissa bits -- see an unbiased rounding, not a
// truncation, without any conversion pass over HBM or shared memory.
//
// Every wait on an mbarrier is bounded: a wait that runs out records ONN_ERR_DEVICE_TIMEOUT
// in a device status word, raises a CTA-wide abort flag that ends all role loops, the
// producer drains the copies it still has in flight, TMEM is freed and the kernel returns.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "gemm_internal.h"
#include "launch_counter.h"
#include "tcgen05.cuh"
#include "work_ring.cuh"

namespace onn
{
namespace tc
{

constexpr int BM = 128;
constexpr int BK = 32;
constexpr int UMMA_K = 8;
constexpr int kThreads = 192;
constexpr int kEpilogueWarps = 4;
constexpr int A_STAGE_BYTES = BM * BK * 4;                 // 16 KiB
constexpr int EPI_BLOCK_BYTES = 32 * 32 * 4;               // one warp's 32 rows x 32 columns
constexpr int EPI_BYTES = kEpilogueWarps * 2 * EPI_BLOCK_BYTES;   // double-buffered per warp: 32 KiB
__device__ int g_selftest_flag;                            // result word of the bounded-wait self-test

struct Params
{
    long long M, N, K;
    long long ldc;
    long long c_stride_inner, c_stride_outer;
    float* C;
    const float* bias;
    const float* relu_mask;
    unsigned int* relu_bits_out;                           // optional: bit n % 32 of word [m][n / 32] = (written value > 0)
    const unsigned int* relu_bits;                         // optional: the same mask, applied to the result
    long long relu_bits_ld;                                // words per row of either bit matrix
    float* colsum;                                         // optional column sums of the written values
    long long colsum_stride_inner;
    float alpha;
    int relu, accumulate;
    int batch_inner, batch_outer;
    int a_batch_inner_on, a_batch_outer_on, b_batch_inner_on, b_batch_outer_on, c_batch_inner_on, c_batch_outer_on;
    int a_wide, b_wide;                                    // MN-major operand loaded with one 5-D box per stage
    int k_parts, k_part_blocks;                            // reduction through k_parts operand pairs of k_part_blocks k-blocks each (two-CTA kernel)
    int splits;
    long long k_per_split;                                 // multiple of BK
    int m_blocks, n_blocks;
    long long total_work;
    // two-CTA kernel only: the last `tail_tiles` tiles of the tile order are each split into two halves of the
    // reduction that two different CTA pairs add into C (see the kernel's header); 0 = no split
    int tail_tiles;
    unsigned long long tail_token;                         // this launch's value of "zeroed" in tail_flags
    unsigned long long* tail_flags;                        // [tail tile][8 epilogue warps of a pair]
    unsigned int* tail_visits;                             // same shape: adders that have seen the token (0, 1, back to 0)
    int sm_cap;                                            // host side: SMs this launch may occupy (read once per launch: the plan and the grid must agree)
    // work items are handed out through this counter in the order the CTAs (CTA pairs) ask for them (it wraps to zero
    // with the last one's question past the end: work_ring.cuh).  A CTA that gets its SM late -- another kernel holds
    // it -- then simply takes fewer items instead of making the whole launch wait for a fixed share.
    // Null: item number t of CTA (pair) q is q + t * grid.
    unsigned int* work_counter;
};

// Instruction descriptor: D = fp32, A = B = tf32, M = 128, N = BN, majors as given.
__host__ __device__ constexpr uint32_t make_idesc(int bn, int a_mn_major, int b_mn_major)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// Work on a staged 32 x 32 output block (row r at r * 128 bytes, 16-byte chunk c at slot c ^ (r % 8)) before it
// is handed to the copy engine:
//   - ReLU mask: the mask block is read with whole 128-byte rows per 8 lanes (4 rows per pass) and applied in place;
//   - column sums: lane L adds up column L over the block's valid rows and issues one reduction per column.
__device__ __forceinline__ void staged_block_passes(const Params& p, uint32_t block, long long warp_row0, long long n_base,
                                                    long long c_offset, int zi, int lane)
{
    if(p.relu_mask)
    {
        // all eight mask loads are issued before anything waits on them
        float4 k[8];
#pragma unroll
        for(int pass = 0; pass < 8; pass++)
        {
            const int r = pass * 4 + (lane >> 3), chunk = lane & 7;
            const long long row = warp_row0 + r, n = n_base + chunk * 4;
            k[pass] = make_float4(1.f, 1.f, 1.f, 1.f);
            if(row < p.M && n < p.N)
            {
                const float* k_ptr = p.relu_mask + c_offset + row * p.ldc + n;
                if(n + 3 < p.N) k[pass] = ld4_stream(k_ptr);
                else { k[pass].x = k_ptr[0]; k[pass].y = n + 1 < p.N ? k_ptr[1] : 0.f; k[pass].z = n + 2 < p.N ? k_ptr[2] : 0.f; k[pass].w = 0.f; }
            }
        }
        __syncwarp();
#pragma unroll
        for(int pass = 0; pass < 8; pass++)
        {
            const int r = pass * 4 + (lane >> 3), chunk = lane & 7;
            const uint32_t at = block + (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4);
            float4 x;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(x.x), "=f"(x.y), "=f"(x.z), "=f"(x.w) : "r"(at));
            x.x = k[pass].x > 0.f ? x.x : 0.f; x.y = k[pass].y > 0.f ? x.y : 0.f;
            x.z = k[pass].z > 0.f ? x.z : 0.f; x.w = k[pass].w > 0.f ? x.w : 0.f;
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(at), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w));
        }
    }
    if(p.colsum)
    {
        __syncwarp();
        const long long left = p.M - warp_row0;
        const int rows_valid = left < 32 ? (int)left : 32;
        float part[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
        for(int r = 0; r < 32; r++)
        {
            const uint32_t at = block + (uint32_t)r * 128u + (uint32_t)(((lane >> 2) ^ (r & 7)) << 4) + (uint32_t)(lane & 3) * 4u;
            float x;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x) : "r"(at));
            part[r & 3] += r < rows_valid ? x : 0.f;
        }
        const float total = (part[0] + part[1]) + (part[2] + part[3]);
        if(n_base + lane < p.N) atomicAdd(p.colsum + (long long)zi * p.colsum_stride_inner + n_base + lane, total);
    }
}

struct WorkItem { int zi, zo, split, m_blk, n_blk; long long k_begin; int k_blocks; int tail; };   // tail: index of a split tail tile, or -1

__device__ __forceinline__ WorkItem decode_work(const Params& p, long long w)
{
    constexpr int kGroup = 8;                               // M blocks per raster group (L2 reuse of B panels)
    const long long tiles = (long long)p.m_blocks * p.n_blocks;
    long long t;
    WorkItem it;
    it.tail = -1;
    if(p.tail_tiles > 0)
    {
        // batch 1, no split-K: whole tiles first, then the two reduction halves of each tail tile, the halves of one
        // tile `tail_tiles` work items apart so that they land on different CTA pairs of the same wave
        const long long whole = tiles - p.tail_tiles;
        it.zi = 0; it.zo = 0;
        const int k_blocks = (int)((p.K + BK - 1) / BK), first_half = (k_blocks + 1) / 2;
        if(w < whole) { t = w; it.split = 0; it.k_begin = 0; it.k_blocks = k_blocks; }
        else
        {
            const long long u = w - whole;
            it.tail = (int)(u % p.tail_tiles);
            it.split = (int)(u / p.tail_tiles);
            t = whole + it.tail;
            it.k_begin = it.split == 0 ? 0 : (long long)first_half * BK;
            it.k_blocks = it.split == 0 ? first_half : k_blocks - first_half;
        }
    }
    else
    {
        t = w % tiles;
        long long rest = w / tiles;
        it.split = (int)(rest % p.splits); rest /= p.splits;
        it.zi = (int)(rest % p.batch_inner);
        it.zo = (int)(rest / p.batch_inner);
    }
    const long long per_group = (long long)kGroup * p.n_blocks;
    const int group = (int)(t / per_group);
    const int first_m = group * kGroup;
    const int group_size = min(p.m_blocks - first_m, kGroup);
    const int in_group = (int)(t % per_group);
    it.m_blk = first_m + in_group % group_size;
    it.n_blk = in_group / group_size;
    if(p.tail_tiles == 0)
    {
        it.k_begin = it.split * p.k_per_split;
        const long long k_end = min(p.K, it.k_begin + p.k_per_split);
        it.k_blocks = (int)((k_end - it.k_begin + BK - 1) / BK);
    }
    return it;
}

// What an epilogue warp fetches for a tile BEFORE it waits for the tile's accumulator: the bias values
// of the tile's columns (lane L holds column 32 j + L) and the ReLU bit words of its rows (lane L holds
// row L, word j covers columns 32 j .. 32 j + 31).  While the operand pipeline keeps the path from L2
// to the SM full, a load issued from the epilogue takes microseconds to return; issued here, that
// time passes behind the tile's MMAs instead of once per 32 x 32 block.
template <int BN>
struct TileSideInputs { float bias[BN / 32]; uint32_t bits[BN / 32]; };

template <int BN>
__device__ __forceinline__ void load_tile_side_inputs(const Params& p, bool use_bias, long long warp_row0, long long n0, int lane,
                                                      TileSideInputs<BN>& side)
{
    const long long row = warp_row0 + lane;
#pragma unroll
    for(int j = 0; j < BN / 32; j++)
    {
        const long long n = n0 + j * 32 + lane;
        side.bias[j] = (use_bias && n < p.N) ? __ldg(p.bias + n) : 0.f;
        side.bits[j] = 0xffffffffu;
        if(p.relu_bits && row < p.M && n0 + j * 32 < p.N) side.bits[j] = __ldg(p.relu_bits + row * p.relu_bits_ld + (n0 >> 5) + j);
    }
}

// One warp's share of one output tile: 32 rows x BN columns from TMEM (lane = row) through the
// alpha / bias / ReLU / mask arithmetic into this warp's two staging blocks and on to C with the copy
// engine.  `warp_blocks` is the shared-memory address of the warp's two 4 KiB blocks; `staged_chunks`
// counts the blocks the warp has handed over so far (it picks the block and tells when to wait).
template <int BN>
__device__ __forceinline__ void epilogue_warp_tile(const Params& p, const CUtensorMap* map_c, uint32_t taddr, uint32_t warp_blocks,
                                                   unsigned int& staged_chunks, long long warp_row0, long long n0,
                                                   long long c_offset, int zi, int c_zi, int c_zo, bool use_bias, bool add_to_c, int lane,
                                                   TileSideInputs<BN>& side)
{
    const bool reduce = p.accumulate || p.splits > 1 || add_to_c;
#pragma unroll 1
    for(int c = 0; c < BN / 32; c++)
    {
        const long long n_base = n0 + c * 32;
        if(n_base >= p.N || warp_row0 >= p.M) break;        // nothing of this block lies inside C
        float v[32];
        __syncwarp();                                       // tcgen05.ld is warp-collective: reconverge first
        tmem_load_32(taddr + c * 32, v);
        // this warp's two staging blocks alternate; a block is free again once the copy issued from it
        // two chunks ago has finished READING shared memory
        const uint32_t block = warp_blocks + (staged_chunks & 1u) * EPI_BLOCK_BYTES;
        if(staged_chunks >= 2) { if(lane == 0) bulk_wait_read_1(); __syncwarp(); }

        const float bias_lane = side.bias[0];               // this block's values; the rest move up one place
        const uint32_t keep = side.bits[0];
#pragma unroll
        for(int j = 0; j + 1 < BN / 32; j++) { side.bias[j] = side.bias[j + 1]; side.bits[j] = side.bits[j + 1]; }

#pragma unroll
        for(int i = 0; i < 32; i++) v[i] *= p.alpha;
        if(use_bias)
        {
#pragma unroll
            for(int i = 0; i < 32; i++) v[i] += __shfl_sync(0xffffffffu, bias_lane, i);
        }
        if(p.relu)
        {
#pragma unroll
            for(int i = 0; i < 32; i++) v[i] = fmaxf(v[i], 0.f);
        }
        if(p.relu_bits)
        {
#pragma unroll
            for(int i = 0; i < 32; i++) v[i] = (keep >> i) & 1u ? v[i] : 0.f;
        }
        if(p.relu_bits_out)
        {
            uint32_t positive = 0;
#pragma unroll
            for(int i = 0; i < 32; i++) positive |= (v[i] > 0.f ? 1u : 0u) << i;
            if(warp_row0 + lane < p.M) p.relu_bits_out[(warp_row0 + lane) * p.relu_bits_ld + (n_base >> 5)] = positive;
        }
#pragma unroll
        for(int q4 = 0; q4 < 8; q4++)
        {
            // row `lane` of the block is 128 bytes; 16-byte chunk q4 goes to slot q4 ^ (lane % 8): the 128-byte swizzle
            const uint32_t dst = block + (uint32_t)lane * 128u + (uint32_t)((q4 ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(dst), "f"(v[q4 * 4]), "f"(v[q4 * 4 + 1]), "f"(v[q4 * 4 + 2]), "f"(v[q4 * 4 + 3]));
        }
        staged_block_passes(p, block, warp_row0, n_base, c_offset, zi, lane);
        fence_async_shared();                               // generic-proxy writes -> visible to the copy engine
        __syncwarp();
        if(lane == 0)
        {
            if(reduce) tma_reduce_add_4d(map_c, block, (int)n_base, (int)warp_row0, c_zi, c_zo);
            else tma_store_4d(map_c, block, (int)n_base, (int)warp_row0, c_zi, c_zo);
            bulk_commit();
        }
        staged_chunks++;
    }
}


template <int BN, int STAGES, int A_MN, int B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const Params p)
{
    constexpr int B_STAGE_BYTES = BN * BK * 4;
    constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;                  // two accumulator buffers (power of two >= 32)
    constexpr uint32_t IDESC = make_idesc(BN, A_MN, B_MN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* epi_smem = smem + (size_t)STAGES * STAGE_BYTES;            // 1024-byte aligned: stage sizes are multiples of 1024
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + EPI_BYTES);
    uint64_t* full_bar = bars;                              // [STAGES]  TMA -> MMA
    uint64_t* empty_bar = bars + STAGES;                    // [STAGES]  MMA -> TMA
    uint64_t* acc_full_bar = bars + 2 * STAGES;             // [2]       MMA -> epilogue
    uint64_t* acc_empty_bar = bars + 2 * STAGES + 2;        // [2]       epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    WorkRing* ring = reinterpret_cast<WorkRing*>(bars + 2 * STAGES + 5);      // producer -> MMA issuer and epilogue warps
    static_assert((2 * STAGES + 5) * 8 + sizeof(WorkRing) <= 256, "barriers beyond their 256 bytes");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < STAGES; s++) { mbar_init(smem_u32(full_bar + s), 1); mbar_init(smem_u32(empty_bar + s), 1); }
        for(int a = 0; a < 2; a++) { mbar_init(smem_u32(acc_full_bar + a), 1); mbar_init(smem_u32(acc_empty_bar + a), kEpilogueWarps); }
        work_ring_init(ring, 1 + kEpilogueWarps);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if(warp == 1)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();                                               // set-up done; global memory only from here on
    // the producer is also the scheduler (work_ring.cuh).  The counter is touched only after the wait: a counter of the
    // pool can come round to two launches that follow each other on the stream
    const WorkSource source = { p.work_counter, (uint32_t)p.total_work, gridDim.x };
    const WorkView work = { ring, p.work_counter != nullptr, (uint32_t)p.total_work };
    uint32_t first_work = kNoWork;
    if(threadIdx.x == 0) first_work = source.fetch(0, blockIdx.x, gridDim.x);

    if(warp == 0)
    {
        // ---------------- TMA producer ----------------
        if(lane == 0)
        {
            uint32_t stage = 0, phase = 0;
            uint32_t armed[STAGES];                          // parity of the last phase armed per stage (+1), 0 = none
#pragma unroll
            for(int s = 0; s < STAGES; s++) armed[s] = 0;
            bool ok = true;
            uint32_t w = first_work;
            ok = work.publish(0, w, abort_flag, 5);
            for(uint32_t turn = 0; ok && w != kNoWork; turn++)
            {
                // item t + 1 is asked for before item t is copied and announced once those copies are on their way
                const uint32_t ahead = source.fetch(turn + 1, blockIdx.x, gridDim.x);
                const WorkItem it = decode_work(p, w);
                const int m0 = it.m_blk * BM, n0 = it.n_blk * BN;
                const int a_zi = p.a_batch_inner_on ? it.zi : 0, a_zo = p.a_batch_outer_on ? it.zo : 0;
                const int b_zi = p.b_batch_inner_on ? it.zi : 0, b_zo = p.b_batch_outer_on ? it.zo : 0;
                for(int kb = 0; kb < it.k_blocks; kb++)
                {
                    if(!mbar_wait(smem_u32(empty_bar + stage), phase ^ 1, abort_flag, 1)) { ok = false; break; }
                    const uint32_t bar = smem_u32(full_bar + stage);
                    const uint32_t a_dst = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                    const uint32_t b_dst = a_dst + A_STAGE_BYTES;
                    const int k0 = (int)(it.k_begin + (long long)kb * BK);
                    mbar_arrive_expect_tx(bar, STAGE_BYTES);
                    armed[stage] = phase + 1;
                    if(A_MN)
                    {
                        if(p.a_wide) tma_load_5d(a_dst, &map_a, bar, 0, k0, m0 / 32, a_zi, a_zo);
                        else
                        {
#pragma unroll
                            for(int j = 0; j < BM / 32; j++) tma_load_4d(a_dst + j * 4096, &map_a, bar, m0 + 32 * j, k0, a_zi, a_zo);
                        }
                    }
                    else
                        tma_load_4d(a_dst, &map_a, bar, k0, m0, a_zi, a_zo);
                    if(B_MN)
                    {
                        if(p.b_wide) tma_load_5d(b_dst, &map_b, bar, 0, k0, n0 / 32, b_zi, b_zo);
                        else
                        {
#pragma unroll
                            for(int j = 0; j < BN / 32; j++) tma_load_4d(b_dst + j * 4096, &map_b, bar, n0 + 32 * j, k0, b_zi, b_zo);
                        }
                    }
                    else
                        tma_load_4d(b_dst, &map_b, bar, k0, n0, b_zi, b_zo);
                    if(++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                w = ahead;
                if(ok) ok = work.publish(turn + 1, w, abort_flag, 5);
            }
            if(*abort_flag)
            {
                // drain: wait (bounded) until every copy this thread started has landed, so that
                // no bulk copy is still writing this CTA's shared memory when it exits
#pragma unroll
                for(int s = 0; s < STAGES; s++)
                    if(armed[s])
                    {
                        const unsigned long long start = clock64();
                        while(!mbar_try_wait(smem_u32(full_bar + s), armed[s] - 1))
                            if(clock64() - start > kWaitCycles) break;
                    }
            }
        }
    }
    else if(warp == 1)
    {
        // ---------------- MMA issuer ----------------
        if(lane == 0)
        {
            uint32_t stage = 0, phase = 0;
            long long local = 0;
            bool ok = true;
            for(uint32_t turn = 0; ok; turn++, local++)
            {
                const uint32_t w = work.take(turn, abort_flag, 6);
                if(w == kNoWork) break;
                const WorkItem it = decode_work(p, w);
                const uint32_t acc = (uint32_t)(local & 1), acc_phase = (uint32_t)((local >> 1) & 1);
                if(!mbar_wait(smem_u32(acc_empty_bar + acc), acc_phase ^ 1, abort_flag, 2)) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for(int kb = 0; kb < it.k_blocks; kb++)
                {
                    if(!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag, 3)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(smem + (size_t)stage * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_STAGE_BYTES;
                    const uint64_t a_desc = A_MN ? make_smem_desc(a_addr, 4096, 512, 1) : make_smem_desc(a_addr, 16, 1024, 2);
                    const uint64_t b_desc = B_MN ? make_smem_desc(b_addr, 4096, 512, 1) : make_smem_desc(b_addr, 16, 1024, 2);
#pragma unroll
                    for(int j = 0; j < BK / UMMA_K; j++)
                    {
                        // descriptor start-address field is in 16-byte units
                        const uint64_t a_step = A_MN ? (uint64_t)(j * 1024 >> 4) : (uint64_t)(j * UMMA_K * 4 >> 4);
                        const uint64_t b_step = B_MN ? (uint64_t)(j * 1024 >> 4) : (uint64_t)(j * UMMA_K * 4 >> 4);
                        tcgen05_mma_tf32(d_tmem, a_desc + a_step, b_desc + b_step, IDESC, (kb > 0 || j > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(smem_u32(empty_bar + stage));     // frees the stage once these MMAs have read it
                    if(++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if(!ok) break;
                tcgen05_commit(smem_u32(acc_full_bar + acc));        // accumulator complete
            }
        }
    }
    else
    {
        // ---------------- epilogue (warps 2..5) ----------------
        const int quadrant = warp & 3;                       // TMEM lanes this warp may read: 32*quadrant ..
        long long local = 0;
        unsigned int staged_chunks = 0;                      // blocks this warp has handed to the copy engine
        for(uint32_t turn = 0; ; turn++, local++)
        {
            const uint32_t w = work.warp_take(turn, lane, abort_flag, 7);
            if(w == kNoWork) break;
            const WorkItem it = decode_work(p, w);
            const uint32_t acc = (uint32_t)(local & 1), acc_phase = (uint32_t)((local >> 1) & 1);
            const long long n0 = (long long)it.n_blk * BN;
            const long long c_offset = it.zi * p.c_stride_inner + it.zo * p.c_stride_outer;
            const bool use_bias = p.bias != nullptr && it.split == 0;
            const long long warp_row0 = (long long)it.m_blk * BM + quadrant * 32;
            TileSideInputs<BN> side;
            load_tile_side_inputs<BN>(p, use_bias, warp_row0, n0, lane, side);

            bool ok = true;
            if(lane == 0) ok = mbar_wait(smem_u32(acc_full_bar + acc), acc_phase, abort_flag, 4);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if(!ok) break;
            tcgen05_fence_after();

            const uint32_t taddr = tmem_base + ((uint32_t)(quadrant * 32) << 16) + acc * BN;
            const int c_zi = p.c_batch_inner_on ? it.zi : 0, c_zo = p.c_batch_outer_on ? it.zo : 0;
            epilogue_warp_tile<BN>(p, &map_c, taddr, smem_u32(epi_smem + (warp - 2) * 2 * EPI_BLOCK_BYTES), staged_chunks, warp_row0, n0,
                                   c_offset, it.zi, c_zi, c_zo, use_bias, false, lane, side);
            tcgen05_fence_before();
            __syncwarp();
            if(lane == 0) mbar_arrive(smem_u32(acc_empty_bar + acc));
        }
        if(lane == 0) bulk_wait_all();                       // the staging blocks must outlive the copies that read them
    }

    tcgen05_fence_before();
    __syncthreads();
    if(warp == 1)
    {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}


// =========================================================================================
// Two-CTA variant (cta_group::2) for the large dense GEMMs.
//
// A cluster of two CTAs on neighbouring SMs computes one 256 x 256 tile: CTA r owns rows
// 128r..128r+127 (its own A tile, its own TMEM accumulator) and stages only HALF of the B tile
// (columns 128r..128r+127); the tensor cores of both SMs read both halves.  Per SM and k-block
// the copy engine writes 32 KB instead of 48 KB and the MMA reads 32 KB instead of 48 KB, which
// lifts the shared-memory-bandwidth ceiling of 4-byte operands from 0.68 to 1.0 of the tensor
// peak, and L2 -> SM operand traffic drops by a third.  No load uses multicast: each CTA copies
// its own halves, with the completion bytes counted on the leader's barrier.
//
// Barriers: full[s] lives in the leader (CTA 0): its producer arms it for the bytes of BOTH
// CTAs, the peer's copies complete on it remotely.  empty[s] and acc_full[b] exist in both CTAs
// and are signalled by the leader's tcgen05.commit to both.  acc_empty[b] lives in the leader
// and counts the epilogue warps of both CTAs.
// =========================================================================================

constexpr int STAGES2 = 6;
constexpr int STAGE2_BYTES = A_STAGE_BYTES + 128 * BK * 4;          // A 16 KiB + half of B 16 KiB

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    return rank;
}

__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}

__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}

// arrival that publishes nothing (a reader handing a ring slot back): no release, so the issuing thread's own work in
// flight -- for the MMA issuer a whole tile of tcgen05.mma -- is not waited for
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}

// bounded wait whose acquire covers what the other CTA of the pair wrote before it arrived on the barrier
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int site)
{
    const unsigned long long start = clock64();
    unsigned int spins = 0;
    while(true)
    {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if(done) return true;
        if((++spins & 255u) == 0)
        {
            if(*abort_flag) return false;
            if(clock64() - start > kWaitCycles)
            {
                atomicCAS(&g_status, 0u, site);
                *abort_flag = 1;
                __threadfence_block();
                return false;
            }
        }
    }
}

constexpr int kTileRing = 4;                                // work items the scheduler may be ahead of the slowest role

// copies of a CTA pair: data lands in the executing CTA, completion bytes go to the barrier at
// `bar` (a shared::cluster address, here always the leader's)
__device__ __forceinline__ void tma2_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tma2_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        :: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}

__device__ __forceinline__ void tcgen05_mma2_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// arrive on the barrier at the same offset in BOTH CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tcgen05_commit2_both(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(bar), "h"((uint16_t)3) : "memory");
}

__host__ __device__ constexpr uint32_t make_idesc2(int a_mn_major, int b_mn_major)
{
    // D = fp32, A = B = tf32, M = 256 (128 rows per CTA), N = 256
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
           ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <int A_MN, int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_c, const Params p)
{
    constexpr int BN = 256;
    constexpr uint32_t TMEM_COLS = 512;                       // two 256-column accumulator buffers per CTA
    constexpr uint32_t IDESC = make_idesc2(A_MN, B_MN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* epi_smem = smem + (size_t)STAGES2 * STAGE2_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + EPI_BYTES);
    uint64_t* full_bar = bars;                                // [STAGES2]  used in the leader only
    uint64_t* empty_bar = bars + STAGES2;                     // [STAGES2]  both CTAs
    uint64_t* acc_full_bar = bars + 2 * STAGES2;              // [2]        both CTAs
    uint64_t* acc_empty_bar = bars + 2 * STAGES2 + 2;         // [2]        used in the leader only
    uint64_t* tile_full_bar = bars + 2 * STAGES2 + 4;         // [kTileRing] both CTAs: the scheduler has written the slot
    uint64_t* tile_empty_bar = tile_full_bar + kTileRing;     // [kTileRing] used in the leader only: every role of both CTAs has read it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tile_empty_bar + kTileRing);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    // [r] = 1 + the number of stage fills the producer of CTA r has started, published to both CTAs when it stops (0 = not yet)
    volatile uint32_t* fills_started = reinterpret_cast<volatile uint32_t*>(tmem_slot + 2);
    volatile uint32_t* tile_ring = reinterpret_cast<volatile uint32_t*>(tmem_slot + 4);   // [kTileRing] work item numbers, kNoWork = the end
    static_assert((2 * STAGES2 + 4 + 2 * kTileRing) * 8 + (4 + kTileRing) * 4 <= 256, "barriers and flags beyond their 256 bytes");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const long long pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if(threadIdx.x == 0)
    {
        for(int s = 0; s < STAGES2; s++) { mbar_init(smem_u32(full_bar + s), 1); mbar_init(smem_u32(empty_bar + s), 1); }
        for(int a = 0; a < 2; a++) { mbar_init(smem_u32(acc_full_bar + a), 1); mbar_init(smem_u32(acc_empty_bar + a), 2 * kEpilogueWarps); }
        // readers of a slot: the MMA issuer and the peer's producer, and the epilogue warps of both CTAs
        for(int r = 0; r < kTileRing; r++) { mbar_init(smem_u32(tile_full_bar + r), 1); mbar_init(smem_u32(tile_empty_bar + r), 2 + 2 * kEpilogueWarps); }
        *abort_flag = 0;
        fills_started[0] = 0; fills_started[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if(warp == 1)
    {
        // both CTAs of the pair run the allocation with the same destination offset
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();                                           // the peer's barriers exist before anyone signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();                                               // set-up done; global memory only from here on
    // the counter is touched only after the wait: a counter of the pool can come round to two launches that follow each
    // other on the stream
    const WorkSource source = { p.work_counter, (uint32_t)p.total_work, (uint32_t)pairs };
    uint32_t first_work = kNoWork;
    if(threadIdx.x == 0 && leader && p.work_counter) first_work = source.fetch(0, 0, 0);

    // Work items.  With a counter the leader's producer thread is the scheduler: it takes item numbers from the counter,
    // one ahead of the item it loads, and publishes each in a ring slot of both CTAs; every other role reads the slots in
    // order (take_item) and frees them on the leader's barrier.  Without one, item number `turn` of this pair is fixed.
    const bool dynamic = p.work_counter != nullptr;
    const auto take_item = [&](uint32_t turn, unsigned int site) -> uint32_t      // one thread per role
    {
        if(!dynamic)
        {
            const long long w = pair + (long long)turn * pairs;
            return w < p.total_work ? (uint32_t)w : kNoWork;
        }
        const uint32_t slot = turn % kTileRing, parity = (turn / kTileRing) & 1u;
        if(!mbar_wait_cluster(smem_u32(tile_full_bar + slot), parity, abort_flag, site)) return kNoWork;
        const uint32_t w = tile_ring[slot];
        // the slot goes back only once its value has arrived in a register (the branch needs it)
        if(w != kNoWork - 1u) mbar_arrive_cluster_relaxed(map_to_cta(smem_u32(tile_empty_bar + slot), 0));
        return w;
    };

    if(warp == 0)
    {
        // ---------------- TMA producer (one per CTA: own A rows, own half of B) ----------------
        if(lane == 0)
        {
            uint32_t stage = 0, phase = 0, fills = 0;
            bool ok = true;
            const bool scheduler = dynamic && leader;
            // the scheduler's next item: asked for one item ahead, so the counter's round trip runs under the copies
            uint32_t ahead = first_work;
            for(uint32_t turn = 0; ok; turn++)
            {
                uint32_t w;
                if(scheduler)
                {
                    const uint32_t slot = turn % kTileRing, parity = (turn / kTileRing) & 1u;
                    if(!mbar_wait(smem_u32(tile_empty_bar + slot), parity ^ 1u, abort_flag, 16)) break;
                    w = ahead;
                    tile_ring[slot] = w;
                    asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(map_to_cta(smem_u32(const_cast<uint32_t*>(tile_ring) + slot), 1)), "r"(w) : "memory");
                    mbar_arrive_cluster(map_to_cta(smem_u32(tile_full_bar + slot), 0));
                    mbar_arrive_cluster(map_to_cta(smem_u32(tile_full_bar + slot), 1));
                    if(w == kNoWork) break;
                    ahead = source.fetch(turn + 1, 0, 0);
                }
                else
                {
                    w = take_item(turn, 17);
                    if(w == kNoWork) break;
                }
                const WorkItem it = decode_work(p, w);
                const int m0 = it.m_blk * 256 + (int)rank * 128, n0 = it.n_blk * BN + (int)rank * 128;
                for(int kb = 0; kb < it.k_blocks; kb++)
                {
                    if(!mbar_wait(smem_u32(empty_bar + stage), phase ^ 1, abort_flag, 11)) { ok = false; break; }
                    const uint32_t bar = map_to_cta(smem_u32(full_bar + stage), 0);      // the leader's barrier
                    const uint32_t a_dst = smem_u32(smem + (size_t)stage * STAGE2_BYTES);
                    const uint32_t b_dst = a_dst + A_STAGE_BYTES;
                    // with several operand pairs the reduction index runs through them one after the other; the pair is the
                    // third coordinate of both maps
                    const int k_block = (int)(it.k_begin / BK) + kb;
                    const int part = p.k_parts > 1 ? k_block / p.k_part_blocks : 0;
                    const int k0 = (p.k_parts > 1 ? k_block % p.k_part_blocks : k_block) * BK;
                    if(leader) mbar_arrive_expect_tx(smem_u32(full_bar + stage), 2 * STAGE2_BYTES);
                    if(A_MN) tma2_load_5d(a_dst, &map_a, bar, 0, k0, m0 / 32, part, 0);
                    else tma2_load_4d(a_dst, &map_a, bar, k0, m0, part, 0);
                    if(B_MN) tma2_load_5d(b_dst, &map_b, bar, 0, k0, n0 / 32, part, 0);
                    else tma2_load_4d(b_dst, &map_b, bar, k0, n0, part, 0);
                    fills++;
                    if(++stage == STAGES2) { stage = 0; phase ^= 1; }
                }
            }
            // Both producers say how many stage fills they started (two stores per kernel).  After a wait has run out
            // that is what lets the pair drain its copies: a fill's bytes of BOTH CTAs complete on the leader's barrier,
            // so a barrier phase only one of them started would never complete and nobody could tell when its copy had
            // landed.  The CTA that is behind therefore starts the fills the other one started (same stages, the
            // first tile's coordinates: the data no longer matters), the leader arms them, and then waits -- bounded --
            // until the last phase started on every stage is complete.  Only then do the CTAs go on to the cluster
            // barrier that precedes the release of tensor memory and the exit.
            fills_started[rank] = fills + 1;
            asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(map_to_cta(smem_u32(const_cast<uint32_t*>(fills_started) + rank), rank ^ 1u)), "r"(fills + 1) : "memory");
            asm volatile("fence.acq_rel.cluster;" ::: "memory");
            if(*abort_flag)
            {
                uint32_t theirs = 0;
                const unsigned long long start = clock64();
                // the partner stops at the latest one wait limit after this CTA did
                while((theirs = fills_started[rank ^ 1u]) == 0 && clock64() - start < 2 * kWaitCycles) { }
                const uint32_t target = theirs > fills + 1 ? theirs - 1 : fills;
                while(fills < target)
                {
                    const uint32_t a_dst = smem_u32(smem + (size_t)stage * STAGE2_BYTES), b_dst = a_dst + A_STAGE_BYTES;
                    const uint32_t bar = map_to_cta(smem_u32(full_bar + stage), 0);
                    if(leader) mbar_arrive_expect_tx(smem_u32(full_bar + stage), 2 * STAGE2_BYTES);
                    if(A_MN) tma2_load_5d(a_dst, &map_a, bar, 0, 0, (int)rank * 4, 0, 0);
                    else tma2_load_4d(a_dst, &map_a, bar, 0, (int)rank * 128, 0, 0);
                    if(B_MN) tma2_load_5d(b_dst, &map_b, bar, 0, 0, (int)rank * 4, 0, 0);
                    else tma2_load_4d(b_dst, &map_b, bar, 0, (int)rank * 128, 0, 0);
                    fills++;
                    if(++stage == STAGES2) { stage = 0; phase ^= 1; }
                }
                if(leader)
                {
                    // fill n uses stage n % STAGES2 in phase (n / STAGES2) & 1: wait for the last fill of every stage
                    for(uint32_t back = 1; back <= (uint32_t)STAGES2 && back <= fills; back++)
                    {
                        const uint32_t n = fills - back;
                        const unsigned long long since = clock64();
                        while(!mbar_try_wait(smem_u32(full_bar + n % STAGES2), (n / STAGES2) & 1u))
                            if(clock64() - since > kWaitCycles) break;
                    }
                }
            }
        }
    }
    else if(warp == 1)
    {
        // ---------------- MMA issuer (leader only) ----------------
        if(lane == 0 && leader)
        {
            uint32_t stage = 0, phase = 0;
            long long local = 0;
            bool ok = true;
            // (Looking the next item up inside the k-block loop, while MMAs are queued, was tried: the extra branch in that
            // loop cost 4-6 % of the kernel, far more than the look-up at the top costs between two tiles.)
            for(uint32_t turn = 0; ok; turn++, local++)
            {
                const uint32_t w = take_item(turn, 18);
                if(w == kNoWork) break;
                const WorkItem it = decode_work(p, w);
                const uint32_t acc = (uint32_t)(local & 1), acc_phase = (uint32_t)((local >> 1) & 1);
                if(!mbar_wait(smem_u32(acc_empty_bar + acc), acc_phase ^ 1, abort_flag, 12)) break;
                tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for(int kb = 0; kb < it.k_blocks; kb++)
                {
                    if(!mbar_wait(smem_u32(full_bar + stage), phase, abort_flag, 13)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(smem + (size_t)stage * STAGE2_BYTES);
                    const uint32_t b_addr = a_addr + A_STAGE_BYTES;
                    const uint64_t a_desc = A_MN ? make_smem_desc(a_addr, 4096, 512, 1) : make_smem_desc(a_addr, 16, 1024, 2);
                    const uint64_t b_desc = B_MN ? make_smem_desc(b_addr, 4096, 512, 1) : make_smem_desc(b_addr, 16, 1024, 2);
#pragma unroll
                    for(int j = 0; j < BK / UMMA_K; j++)
                    {
                        const uint64_t a_step = A_MN ? (uint64_t)(j * 1024 >> 4) : (uint64_t)(j * UMMA_K * 4 >> 4);
                        const uint64_t b_step = B_MN ? (uint64_t)(j * 1024 >> 4) : (uint64_t)(j * UMMA_K * 4 >> 4);
                        tcgen05_mma2_tf32(d_tmem, a_desc + a_step, b_desc + b_step, IDESC, (kb > 0 || j > 0) ? 1u : 0u);
                    }
                    tcgen05_commit2_both(smem_u32(empty_bar + stage));     // frees this stage in both CTAs
                    if(++stage == STAGES2) { stage = 0; phase ^= 1; }
                }
                if(!ok) break;
                tcgen05_commit2_both(smem_u32(acc_full_bar + acc));         // accumulators complete in both CTAs
            }
        }
    }
    else
    {
        // ---------------- epilogue (warps 2..5 of each CTA, its own 128 rows) ----------------
        const int quadrant = warp & 3;
        long long local = 0;
        unsigned int staged_chunks = 0;
        const uint32_t leader_acc_empty = map_to_cta(smem_u32(acc_empty_bar), 0);
        const uint32_t warp_blocks = smem_u32(epi_smem + (warp - 2) * 2 * EPI_BLOCK_BYTES);
        const int flag_slot = (int)rank * 4 + quadrant;      // this warp's place among the 8 epilogue warps of a pair

        // Split tail tiles are ADDED into by two pairs, so C must hold zeros there first (unless the caller's values
        // are to be kept).  Whoever takes work item j < tail_tiles -- among the first items handed out -- zeroes tail
        // tile j before it turns to the item itself: each warp its own 32 rows, from one zero-filled staging block, and
        // publishes that under this launch's token; the adding warps look the token up before their first reduce
        // (the tail items are the last of the order: the look-up never waits in practice, it is there so that the order
        // is guaranteed rather than likely).
        const auto zero_tail_tile = [&](long long j)
        {
            const long long whole = (long long)p.m_blocks * p.n_blocks - p.tail_tiles;
            Params q = p;                                   // decode the tile itself, not one of its halves
            q.tail_tiles = 0; q.splits = 1; q.batch_inner = 1; q.k_per_split = p.K;
            const WorkItem tile = decode_work(q, whole + j);
            const long long rows0 = (long long)tile.m_blk * 256 + (long long)rank * 128 + quadrant * 32;
            if(lane == 0) bulk_wait_read_0();               // the staging block may still be the source of an earlier store
            __syncwarp();
#pragma unroll
            for(int q4 = 0; q4 < 8; q4++)
            {
                const uint32_t dst = warp_blocks + (uint32_t)lane * 128u + (uint32_t)(q4 << 4);
                asm volatile("st.shared.v4.f32 [%0], {%1, %1, %1, %1};" :: "r"(dst), "f"(0.f));
            }
            fence_async_shared();
            __syncwarp();
            if(lane == 0)
            {
                if(rows0 < p.M)
                    for(int c = 0; c < BN / 32; c++)
                        if((long long)tile.n_blk * BN + c * 32 < p.N) tma_store_4d(&map_c, warp_blocks, tile.n_blk * BN + c * 32, (int)rows0, 0, 0);
                bulk_commit();
                bulk_wait_all();                            // the zeros are in memory, not just on their way
                asm volatile("fence.proxy.async;" ::: "memory");
                __threadfence();
                asm volatile("st.release.gpu.global.u64 [%0], %1;" :: "l"(p.tail_flags + j * 8 + flag_slot), "l"(p.tail_token) : "memory");
            }
            __syncwarp();
        };

        for(uint32_t turn = 0; ; turn++, local++)
        {
            uint32_t w = 0;
            if(lane == 0) w = take_item(turn, 19);
            w = __shfl_sync(0xffffffffu, w, 0);
            if(w == kNoWork) break;
            if(p.tail_tiles > 0 && !p.accumulate && w < (uint32_t)p.tail_tiles) zero_tail_tile(w);
            const WorkItem it = decode_work(p, w);
            const uint32_t acc = (uint32_t)(local & 1), acc_phase = (uint32_t)((local >> 1) & 1);
            const long long n0 = (long long)it.n_blk * BN;
            const bool use_bias = p.bias != nullptr && it.split == 0;
            const long long warp_row0 = (long long)it.m_blk * 256 + (long long)rank * 128 + quadrant * 32;
            TileSideInputs<BN> side;
            load_tile_side_inputs<BN>(p, use_bias, warp_row0, n0, lane, side);
            if(it.tail >= 0 && !p.accumulate)
            {
                // this strip of the tail tile has been zeroed (see above) before anything is added to it
                bool zeroed = true;
                if(lane == 0)
                {
                    const unsigned long long* flag = p.tail_flags + (long long)it.tail * 8 + flag_slot;
                    const unsigned long long start = clock64();
                    unsigned long long seen;
                    while(true)
                    {
                        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(flag) : "memory");
                        if(seen == p.tail_token) break;
                        if(*abort_flag || clock64() - start > kWaitCycles) { atomicCAS(&g_status, 0u, 15u); *abort_flag = 1; zeroed = false; break; }
                    }
                    asm volatile("fence.proxy.async;" ::: "memory");
                    // the second of the strip's two adders to get here clears the token, so that a replay of this very
                    // launch (a captured graph carries the same token) starts from "not zeroed" again
                    unsigned int* visits = p.tail_visits + (long long)it.tail * 8 + flag_slot;
                    if(zeroed && atomicAdd(visits, 1u) == 1u)
                    {
                        *visits = 0u;
                        asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(flag), "l"(0ull) : "memory");
                    }
                }
                zeroed = __shfl_sync(0xffffffffu, zeroed, 0);
                if(!zeroed) break;
            }

            bool ok = true;
            if(lane == 0) ok = mbar_wait(smem_u32(acc_full_bar + acc), acc_phase, abort_flag, 14);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if(!ok) break;
            tcgen05_fence_after();

            const uint32_t taddr = tmem_base + ((uint32_t)(quadrant * 32) << 16) + acc * BN;
            epilogue_warp_tile<BN>(p, &map_c, taddr, warp_blocks, staged_chunks, warp_row0, n0,
                                   0, 0, 0, 0, use_bias, it.tail >= 0, lane, side);
            tcgen05_fence_before();
            __syncwarp();
            if(lane == 0) mbar_arrive_cluster(leader_acc_empty + acc * 8);     // one arrival per epilogue warp of the pair
        }
        if(lane == 0) bulk_wait_all();
    }

    // nobody leaves while the partner may still read this CTA's shared memory or signal its barriers
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();
    if(warp == 1)
    {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}


// Self-test of the bounded wait: a barrier that nothing ever arrives on, waited for with a 1 ms limit.
// The wait must give up, record its site in the status word and let the kernel return normally.
__global__ void bounded_wait_selftest_kernel(int* gave_up)
{
    __shared__ uint64_t never_signalled;
    __shared__ int abort_flag;
    if(threadIdx.x == 0)
    {
        abort_flag = 0;
        mbar_init(smem_u32(&never_signalled), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool completed = mbar_wait(smem_u32(&never_signalled), 0, &abort_flag, 99, 1ull << 21);
        *gave_up = completed ? 0 : 1;
    }
}

// ---- host side --------------------------------------------------------------------------

static bool mult4(long long x) { return (x & 3) == 0; }

template <int BN, int STAGES, int A_MN, int B_MN>
static int launch_variant(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c, const Params& p, cudaStream_t stream)
{
    constexpr int smem = STAGES * (A_STAGE_BYTES + BN * BK * 4) + EPI_BYTES + 1024 + 256;
    static PerDeviceBytes configured;                        // per instantiation and per device
    if(!ensure_dynamic_smem(gemm_tc_kernel<BN, STAGES, A_MN, B_MN>, configured, smem)) return ONN_ERR_CUDA;
    const long long cap = (long long)p.sm_cap * (BN == 64 ? 2 : 1);
    const int grid = (int)(p.total_work < cap ? p.total_work : cap);
    const cudaError_t launched = launch_overlapped(gemm_tc_kernel<BN, STAGES, A_MN, B_MN>, dim3(grid), dim3(kThreads), smem, stream, map_a, map_b, map_c, p);
    count_launch();
    return launched == cudaSuccess ? launch_status() : ONN_ERR_CUDA;
}

template <int A_MN, int B_MN>
static int launch_majors(int bn, const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c, const Params& p, cudaStream_t stream)
{
    if(bn == 256) return launch_variant<256, 4, A_MN, B_MN>(map_a, map_b, map_c, p, stream);
    if(bn == 128) return launch_variant<128, 6, A_MN, B_MN>(map_a, map_b, map_c, p, stream);
    return launch_variant<64, 3, A_MN, B_MN>(map_a, map_b, map_c, p, stream);
}


template <int A_MN, int B_MN>
static int launch_pair_variant(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c, const Params& p, cudaStream_t stream)
{
    constexpr int smem = STAGES2 * STAGE2_BYTES + EPI_BYTES + 1024 + 256;
    static PerDeviceBytes configured;                        // per instantiation and per device
    if(!ensure_dynamic_smem(gemm_tc2_kernel<A_MN, B_MN>, configured, smem)) return ONN_ERR_CUDA;
    const long long pairs_cap = p.sm_cap / 2;
    const long long pairs = p.total_work < pairs_cap ? p.total_work : pairs_cap;
    const cudaError_t launched = launch_overlapped(gemm_tc2_kernel<A_MN, B_MN>, dim3((unsigned)(2 * pairs)), dim3(kThreads), smem, stream, map_a, map_b, map_c, p);
    count_launch();
    return launched == cudaSuccess ? launch_status() : ONN_ERR_CUDA;
}

}  // namespace tc

namespace tc
{
// "zeroed" tokens of split tail tiles: kTailFlagSets launches may be in flight at once without sharing a set
constexpr int kTailFlagSets = 16;
constexpr int kTailFlagsPerSet = (kSmCount / 2) * 8;
static __device__ unsigned long long g_tail_flags[kTailFlagSets * kTailFlagsPerSet];
static __device__ unsigned int g_tail_visits[kTailFlagSets * kTailFlagsPerSet];

static int tail_flags_for_current_device(unsigned long long** flags, unsigned int** visits)
{
    static std::mutex mutex;
    static unsigned long long* resolved_flags[kMaxDevices] = {};
    static unsigned int* resolved_visits[kMaxDevices] = {};
    int device = -1;
    if(cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return ONN_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mutex);
    if(!resolved_flags[device])
    {
        unsigned long long* found_flags = nullptr;
        unsigned int* found_visits = nullptr;
        if(cudaGetSymbolAddress(reinterpret_cast<void**>(&found_flags), g_tail_flags) != cudaSuccess || !found_flags) return ONN_ERR_CUDA;
        if(cudaGetSymbolAddress(reinterpret_cast<void**>(&found_visits), g_tail_visits) != cudaSuccess || !found_visits) return ONN_ERR_CUDA;
        resolved_flags[device] = found_flags;
        resolved_visits[device] = found_visits;
    }
    *flags = resolved_flags[device];
    *visits = resolved_visits[device];
    return ONN_OK;
}
}  // namespace tc

bool gemm_tc_supported(const onn_gemm_args& g)
{
    using tc::mult4;
    if(g.a_major == 1 && g.b_major == 0) return false;      // combination no layer needs
    if(!host_aligned16(g.A) || !host_aligned16(g.B) || !host_aligned16(g.C)) return false;
    if(!mult4(g.lda) || !mult4(g.ldb) || !mult4(g.ldc)) return false;
    if(!mult4(g.a_stride_inner) || !mult4(g.a_stride_outer) || !mult4(g.b_stride_inner) || !mult4(g.b_stride_outer)) return false;
    if(!mult4(g.c_stride_inner) || !mult4(g.c_stride_outer)) return false;
    if(g.bias && !host_aligned16(g.bias)) return false;
    if(g.relu_mask && !host_aligned16(g.relu_mask)) return false;
    if(g.M >= (1LL << 31) || g.N >= (1LL << 31) || g.K >= (1LL << 31)) return false;
    return tc::encode_tiled() != nullptr;
}

static bool pair_kernel_takes(const onn_gemm_args& g)
{
    static const bool pair_enabled = []{ const char* e = std::getenv("ONN_B200_GEMM_PAIR"); return !(e && e[0] == '0'); }();
    return pair_enabled && g.batch_inner == 1 && g.batch_outer == 1 && g.M >= 512 && g.N >= 256 &&
           (g.a_major == 0 || g.M % 32 == 0) && (g.b_major == 0 || g.N % 32 == 0);
}

bool gemm_tc_takes_parts(const onn_gemm_args& g)
{
    using tc::mult4;
    return gemm_tc_supported(g) && pair_kernel_takes(g) && g.K % tc::BK == 0 && g.a_stride_part != 0 && g.b_stride_part != 0 &&
           mult4(g.a_stride_part) && mult4(g.b_stride_part);
}

int gemm_tc_launch(const onn_gemm_args& g, cudaStream_t stream)
{
    using namespace tc;
    const int bn = g.N > 128 ? 256 : (g.N > 64 ? 128 : 64);

    const int parts = g.k_parts > 1 ? g.k_parts : 1;
    Params p;
    p.M = g.M; p.N = g.N; p.K = g.K * parts; p.ldc = g.ldc;
    p.k_parts = parts; p.k_part_blocks = (int)(g.K / BK);
    p.c_stride_inner = g.c_stride_inner; p.c_stride_outer = g.c_stride_outer;
    p.C = g.C; p.bias = g.bias; p.relu_mask = g.relu_mask; p.alpha = g.alpha;
    p.relu_bits_out = g.relu_bits_out; p.relu_bits = g.relu_bits; p.relu_bits_ld = g.relu_bits_ld;
    p.colsum = g.colsum_out; p.colsum_stride_inner = g.colsum_stride_inner;
    p.tail_tiles = 0; p.tail_token = 0; p.tail_flags = nullptr; p.tail_visits = nullptr;
    p.work_counter = nullptr;
    p.sm_cap = sm_limit();
    p.relu = g.relu; p.accumulate = (g.flags & ONN_ACCUMULATE) != 0;
    p.batch_inner = g.batch_inner; p.batch_outer = g.batch_outer;
    p.a_batch_inner_on = g.batch_inner > 1 && g.a_stride_inner != 0; p.a_batch_outer_on = g.batch_outer > 1 && g.a_stride_outer != 0;
    p.b_batch_inner_on = g.batch_inner > 1 && g.b_stride_inner != 0; p.b_batch_outer_on = g.batch_outer > 1 && g.b_stride_outer != 0;
    p.c_batch_inner_on = g.batch_inner > 1 && g.c_stride_inner != 0; p.c_batch_outer_on = g.batch_outer > 1 && g.c_stride_outer != 0;

    p.a_wide = g.a_major == 1 && g.M % 32 == 0;
    p.b_wide = g.b_major == 1 && g.N % 32 == 0;

    const long long k_blocks = (p.K + BK - 1) / BK;
    long long splits = g.split_k > 1 ? g.split_k : 1;
    if(splits > k_blocks) splits = k_blocks;
    const long long blocks_per_split = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + blocks_per_split - 1) / blocks_per_split;   // every split owns at least one k-block
    p.splits = (int)splits;
    p.k_per_split = blocks_per_split * BK;
    p.m_blocks = (int)((g.M + BM - 1) / BM);
    p.n_blocks = (int)((g.N + bn - 1) / bn);
    p.total_work = (long long)p.m_blocks * p.n_blocks * splits * g.batch_inner * g.batch_outer;

    CUtensorMap map_a, map_b, map_c;
    bool ok;

    // large single GEMMs go to the two-CTA kernel (256 x 256 tiles per CTA pair)
    const bool pair = pair_kernel_takes(g);
    if(!pair && parts > 1) return ONN_ERR_UNSUPPORTED;       // the front end only sends operand pairs the two-CTA kernel takes
    if(pair)
    {
        p.m_blocks = (int)((g.M + 255) / 256);
        p.n_blocks = (int)((g.N + 255) / 256);
        p.total_work = (long long)p.m_blocks * p.n_blocks * splits;
        // a last wave that is at most half full is split in two along the reduction (linear epilogues only)
        static const bool tail_split_enabled = []{ const char* e = std::getenv("ONN_B200_GEMM_TAIL_SPLIT"); return !(e && e[0] == '0'); }();
        const long long tiles = (long long)p.m_blocks * p.n_blocks, pairs_cap = p.sm_cap / 2, tail = tiles % pairs_cap;
        if(tail_split_enabled && splits == 1 && tiles > pairs_cap && tail > 0 && 2 * tail <= pairs_cap && k_blocks >= 16 &&
           !g.relu && !g.relu_mask && !g.relu_bits && !g.relu_bits_out)
        {
            unsigned long long* flags = nullptr;
            unsigned int* visits = nullptr;
            if(tail_flags_for_current_device(&flags, &visits) == ONN_OK)
            {
                static std::atomic<unsigned long long> sequence{0};
                const unsigned long long token = ++sequence;
                p.tail_tiles = (int)tail;
                p.tail_token = token;
                p.tail_flags = flags + (token % kTailFlagSets) * kTailFlagsPerSet;
                p.tail_visits = visits + (token % kTailFlagSets) * kTailFlagsPerSet;
                p.total_work = tiles + tail;
            }
        }
        // work items through a counter (null: a fixed share per CTA pair)
        if(p.total_work + pairs_cap < (1LL << 31)) p.work_counter = next_work_counter();
        if(g.a_major == 0) ok = make_map(&map_a, g.A, g.K, g.M, g.lda, parts, g.a_stride_part, 1, 0, BK, BM, false);
        else ok = make_wide_map(&map_a, g.A, g.M, g.K, g.lda, parts, g.a_stride_part, 1, 0, BM / 32, BK);
        if(g.b_major == 0) ok = ok && make_map(&map_b, g.B, g.K, g.N, g.ldb, parts, g.b_stride_part, 1, 0, BK, 128, false);
        else ok = ok && make_wide_map(&map_b, g.B, g.N, g.K, g.ldb, parts, g.b_stride_part, 1, 0, 128 / 32, BK);
        ok = ok && make_map(&map_c, g.C, g.N, g.M, g.ldc, 1, 0, 1, 0, 32, 32, false, false);
        if(!ok) return ONN_ERR_UNSUPPORTED;
        if(g.a_major == 0 && g.b_major == 0) return launch_pair_variant<0, 0>(map_a, map_b, map_c, p, stream);
        if(g.a_major == 0 && g.b_major == 1) return launch_pair_variant<0, 1>(map_a, map_b, map_c, p, stream);
        return launch_pair_variant<1, 1>(map_a, map_b, map_c, p, stream);
    }

    if(g.a_major == 0) ok = make_map(&map_a, g.A, g.K, g.M, g.lda, g.batch_inner, g.a_stride_inner, g.batch_outer, g.a_stride_outer, BK, BM, false);
    else if(p.a_wide) ok = make_wide_map(&map_a, g.A, g.M, g.K, g.lda, g.batch_inner, g.a_stride_inner, g.batch_outer, g.a_stride_outer, BM / 32, BK);
    else ok = make_map(&map_a, g.A, g.M, g.K, g.lda, g.batch_inner, g.a_stride_inner, g.batch_outer, g.a_stride_outer, 32, BK, true);
    if(g.b_major == 0) ok = ok && make_map(&map_b, g.B, g.K, g.N, g.ldb, g.batch_inner, g.b_stride_inner, g.batch_outer, g.b_stride_outer, BK, bn, false);
    else if(p.b_wide) ok = ok && make_wide_map(&map_b, g.B, g.N, g.K, g.ldb, g.batch_inner, g.b_stride_inner, g.batch_outer, g.b_stride_outer, bn / 32, BK);
    else ok = ok && make_map(&map_b, g.B, g.N, g.K, g.ldb, g.batch_inner, g.b_stride_inner, g.batch_outer, g.b_stride_outer, 32, BK, true);
    // C: 32 x 32 blocks, plain fp32 (no rounding), 128-byte swizzle to match the staging layout
    ok = ok && make_map(&map_c, g.C, g.N, g.M, g.ldc, g.batch_inner, g.c_stride_inner, g.batch_outer, g.c_stride_outer, 32, 32, false, false);
    if(!ok) return ONN_ERR_UNSUPPORTED;

    if(p.total_work + 2 * kSmCount < (1LL << 31)) p.work_counter = next_work_counter();
    if(g.a_major == 0 && g.b_major == 0) return launch_majors<0, 0>(bn, map_a, map_b, map_c, p, stream);
    if(g.a_major == 0 && g.b_major == 1) return launch_majors<0, 1>(bn, map_a, map_b, map_c, p, stream);
    if(g.a_major == 1 && g.b_major == 1) return launch_majors<1, 1>(bn, map_a, map_b, map_c, p, stream);
    return ONN_ERR_UNSUPPORTED;
}

int gemm_tc_bounded_wait_selftest(int* gave_up_host)
{
    int* flag = nullptr;
    if(cudaGetSymbolAddress(reinterpret_cast<void**>(&flag), tc::g_selftest_flag) != cudaSuccess) return ONN_ERR_CUDA;
    tc::bounded_wait_selftest_kernel<<<1, 32>>>(flag);
    count_launch();
    if(cudaDeviceSynchronize() != cudaSuccess) return ONN_ERR_CUDA;
    if(cudaMemcpy(gave_up_host, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ONN_ERR_CUDA;
    return ONN_OK;
}

const unsigned int* gemm_tc_status_word() { return tc::status_word_address(); }

int gemm_tc_read_status()
{
    unsigned int status = 0;
    if(tc::read_and_clear_status(&status) != 0) return ONN_ERR_CUDA;
    return status == 0 ? ONN_OK : ONN_ERR_DEVICE_TIMEOUT;
}

}  // namespace onn
