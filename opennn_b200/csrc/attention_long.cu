// Attention core for source lengths above 256 (head size 64): the fused kernels of attention_tc.cu walked over the
// keys in tiles of 256, so that the [Sq, Sk] score matrix still crosses HBM only as the attention weights the layer
// keeps (forward: written once; backward: read once, and the score gradient written once).
// Replaces, for these shapes, the scores GEMM -> mask + softmax kernel -> context GEMM sequence (and its backward),
// i.e. opennn/multihead_attention_layer.cpp:699-756 (forward) and :843-887 (backward) of the reference's CUDA path.
//
// Forward, per (batch, head, 128-query tile): the softmax of a row needs the maximum and the sum over ALL its keys
// before any weight can be written, and the weights must leave normalised.  So the keys are walked twice.  Sweep 1
// computes S = Q K^T tile by tile on the tensor cores and only keeps each row's running maximum and sum (rescaled when
// the maximum moves); sweep 2 computes the tiles again, turns them into exp(s - max) with the FINAL maximum, writes the
// normalised weights, and feeds the unnormalised, tf32-rounded exponentials from tensor memory into the context MMAs,
// which accumulate O over the key tiles; O is normalised once at the end.  The second score product costs tensor-core
// time the kernel has to spare (it is bound by writing the weights) and K comes from L2 the second time.
// Key tiles that the causal mask removes entirely are skipped in both sweeps; their weights are written as zeros.
//
// Backward: dP = dO V^T, dS = P * (dP - delta) with delta = rowsum(dO * O) (needs no P), dQ = scale * sum over key tiles
// of dS K, accumulated in tensor memory.  One sweep; V and K of a tile share one buffer (K arrives when the dP MMAs
// have read V).
//
// Roles, tensor-memory layout, staging and the bounded waits are those of attention_tc.cu.
#include <cmath>

#include "attention_internal.h"
#include "attention_parts.cuh"
#include "common.cuh"
#include "launch_counter.h"
#include "tcgen05.cuh"

namespace onn
{
namespace tc
{

__device__ __forceinline__ int live_key_tiles(const AttnParams& p, int q_tile)
{
    if(!p.causal) return p.key_tiles;
    const int last_query = q_tile * kQRows + kQRows - 1;
    const int tiles = last_query / kMaxKeys + 1;
    return tiles < p.key_tiles ? tiles : p.key_tiles;
}

__device__ __forceinline__ void drain_phase(uint64_t* bar, int parity)
{
    if(parity < 0) return;
    const unsigned long long start = clock64();
    while(!mbar_try_wait(smem_u32(bar), (uint32_t)parity))
        if(clock64() - start > kWaitCycles) break;
}

constexpr int kLongSmem = 2 * (kQRows + 2 * kMaxKeys) * 128 + kSoftmaxWarps * 2 * kBlock + 2 * kQRows * 4 + 1024 + 512;
static_assert(kLongSmem <= 232448, "beyond the shared memory of one CTA");

// ---------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_long_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_p,
                          const __grid_constant__ CUtensorMap map_ctx, const AttnParams p)
{
    constexpr int KB = HD / 32;
    constexpr int Q_BYTES = KB * kQRows * 128;
    constexpr int K_BYTES = KB * kMaxKeys * 128;
    constexpr int V_BYTES = KB * kMaxKeys * 128;
    constexpr uint32_t TMEM_COLS = 512;                     // scores 0..255, context 256..256+HD
    constexpr uint32_t O_COL = kMaxKeys;
    constexpr uint32_t IDESC_O = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(kQRows >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem;
    uint8_t* k_smem = q_smem + Q_BYTES;
    uint8_t* v_smem = k_smem + K_BYTES;
    uint8_t* stage_smem = v_smem + V_BYTES;
    float* exchange = reinterpret_cast<float*>(stage_smem + kSoftmaxWarps * 2 * kBlock);     // [2 halves][128 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(exchange + 2 * kQRows);
    uint64_t* qk_full = bars + 0;
    uint64_t* v_full = bars + 1;
    uint64_t* qk_empty = bars + 2;
    uint64_t* v_empty = bars + 3;
    uint64_t* s_full = bars + 4;
    uint64_t* p_ready = bars + 5;
    uint64_t* o_full = bars + 6;
    uint64_t* o_free = bars + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if(threadIdx.x == 0)
    {
        mbar_init(smem_u32(qk_full), 1); mbar_init(smem_u32(v_full), 1);
        mbar_init(smem_u32(qk_empty), 1); mbar_init(smem_u32(v_empty), 1);
        mbar_init(smem_u32(s_full), 1); mbar_init(smem_u32(o_full), 1);
        mbar_init(smem_u32(p_ready), kSoftmaxWarps); mbar_init(smem_u32(o_free), kSoftmaxWarps);
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

    // Every role walks the same sequence of steps: for each item, sweep 0 then sweep 1 over its live key tiles.
    // n counts steps, n2 the steps of sweep 1 (the ones with V and a context MMA), both give barrier parities.
    if(warp == 0)
    {
        // ---------------- TMA producer ----------------
        if(lane == 0)
        {
            uint32_t n = 0, n2 = 0;
            int qk_armed = -1, v_armed = -1;
            bool ok = true;
            for(long long w = blockIdx.x; ok && w < p.items; w += gridDim.x)
            {
                const AttnItem it = decode_item(p, w);
                const int live = live_key_tiles(p, it.q_tile);
                for(int sweep = 0; ok && sweep < 2; sweep++)
                    for(int kt = 0; kt < live; kt++)
                    {
                        // Q (first step of the item) and K may be replaced once the previous step's score MMAs have read them
                        if(!mbar_wait(smem_u32(qk_empty), (n & 1u) ^ 1u, abort_flag, 41)) { ok = false; break; }
                        const bool first = sweep == 0 && kt == 0;
                        mbar_arrive_expect_tx(smem_u32(qk_full), (first ? Q_BYTES : 0) + K_BYTES);
                        qk_armed = (int)(n & 1u);
#pragma unroll
                        for(int kb = 0; kb < KB; kb++)
                        {
                            if(first) tma_load_4d(smem_u32(q_smem + kb * kQRows * 128), &map_q, smem_u32(qk_full), it.h * HD + kb * 32, it.q_tile * kQRows, 0, it.b);
                            tma_load_4d(smem_u32(k_smem + kb * kMaxKeys * 128), &map_k, smem_u32(qk_full), it.h * HD + kb * 32, kt * kMaxKeys, 0, it.b);
                        }
                        n++;
                        if(sweep == 1)
                        {
                            // V's buffer is free once the previous context MMAs are done
                            if(!mbar_wait(smem_u32(v_empty), (n2 & 1u) ^ 1u, abort_flag, 42)) { ok = false; break; }
                            mbar_arrive_expect_tx(smem_u32(v_full), V_BYTES);
                            v_armed = (int)(n2 & 1u);
                            tma_load_5d(smem_u32(v_smem), &map_v, smem_u32(v_full), 0, kt * kMaxKeys, it.h * KB, 0, it.b);
                            n2++;
                        }
                    }
            }
            if(*abort_flag)
            {
                // no copy may still be writing this CTA's shared memory when it exits
                drain_phase(qk_full, qk_armed);
                drain_phase(v_full, v_armed);
            }
        }
    }
    else if(warp == 1)
    {
        // ---------------- MMA issuer ----------------
        if(lane == 0)
        {
            uint32_t n = 0, n2 = 0, items_done = 0;
            bool ok = true;
            for(long long w = blockIdx.x; ok && w < p.items; w += gridDim.x, items_done++)
            {
                const AttnItem it = decode_item(p, w);
                const int live = live_key_tiles(p, it.q_tile);
                for(int sweep = 0; ok && sweep < 2; sweep++)
                    for(int kt = 0; kt < live; kt++)
                    {
                        const int keys = min(kMaxKeys, p.Sk - kt * kMaxKeys);
                        const int blocks = (keys + 31) / 32;
                        const uint32_t idesc_s = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)((blocks * 32) >> 3) << 17) | ((uint32_t)(kQRows >> 4) << 24);
                        // the tensor pipe runs in order: the previous step's context MMAs (which read the exponentials from the
                        // score columns) were issued before these score MMAs overwrite them
                        if(!mbar_wait(smem_u32(qk_full), n & 1u, abort_flag, 43)) { ok = false; break; }
                        tcgen05_fence_after();
#pragma unroll
                        for(int kb = 0; kb < KB; kb++)
                        {
                            const uint64_t a_desc = make_smem_desc(smem_u32(q_smem + kb * kQRows * 128), 16, 1024, 2);
                            const uint64_t b_desc = make_smem_desc(smem_u32(k_smem + kb * kMaxKeys * 128), 16, 1024, 2);
#pragma unroll
                            for(int j = 0; j < 4; j++)
                                tcgen05_mma_tf32(tmem_base, a_desc + (uint64_t)(j * 32 >> 4), b_desc + (uint64_t)(j * 32 >> 4), idesc_s, (kb > 0 || j > 0) ? 1u : 0u);
                        }
                        tcgen05_commit(smem_u32(qk_empty));           // Q and K may be overwritten
                        tcgen05_commit(smem_u32(s_full));             // scores complete
                        // sweep 0: the softmax threads hold the scores in registers; sweep 1: the exponentials are in tensor memory
                        if(!mbar_wait(smem_u32(p_ready), n & 1u, abort_flag, 44)) { ok = false; break; }
                        n++;
                        if(sweep == 1)
                        {
                            if(!mbar_wait(smem_u32(v_full), n2 & 1u, abort_flag, 45)) { ok = false; break; }
                            // the previous item's context has been read out of the accumulator
                            if(kt == 0 && !mbar_wait(smem_u32(o_free), (items_done & 1u) ^ 1u, abort_flag, 46)) { ok = false; break; }
                            tcgen05_fence_after();
                            const uint64_t v_desc = make_smem_desc(smem_u32(v_smem), kMaxKeys * 128, 512, 1);
                            const int k_steps = blocks * 4;          // 8 keys per MMA
                            for(int kk = 0; kk < k_steps; kk++)
                                tcgen05_mma_tf32_a_tmem(tmem_base + O_COL, tmem_base + (uint32_t)(kk * 8), v_desc + (uint64_t)(kk * 1024 >> 4), IDESC_O,
                                                        (kt > 0 || kk > 0) ? 1u : 0u);
                            tcgen05_commit(smem_u32(v_empty));
                            if(kt == live - 1) tcgen05_commit(smem_u32(o_full));
                            n2++;
                        }
                    }
            }
        }
    }
    else
    {
        // ---------------- softmax and output (warps 2..9) ----------------
        const int quadrant = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r_local = quadrant * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quadrant * 32) << 16);
        const uint32_t warp_blocks = smem_u32(stage_smem + (warp - 2) * 2 * kBlock);
        const float to_log2 = p.scale * kLog2e;
        unsigned int staged = 0;
        uint32_t n = 0, items_done = 0;
        bool ok = true;
        for(long long w = blockIdx.x; ok && w < p.items; w += gridDim.x, items_done++)
        {
            const AttnItem it = decode_item(p, w);
            const int live = live_key_tiles(p, it.q_tile);
            const int row0 = it.q_tile * kQRows + quadrant * 32;
            const int q_row = row0 + lane;
            float run_max = -INFINITY, run_sum = 0.f;        // this thread's half of the row, over the key tiles of sweep 0
            float row_max = 0.f, inv = 0.f;                  // of the whole row, known after sweep 0

            for(int sweep = 0; ok && sweep < 2; sweep++)
                for(int kt = 0; kt < live; kt++)
                {
                    const int tile_key0 = kt * kMaxKeys + half * kHalfKeys;
                    uint32_t pad_word[4];
#pragma unroll
                    for(int j = 0; j < 4; j++)
                    {
                        const int key = tile_key0 + j * 32 + lane;
                        const bool flag = p.key_is_pad && key < p.Sk && p.key_is_pad[(long long)it.b * p.Sk + key] != 0;
                        pad_word[j] = __ballot_sync(0xffffffffu, flag);
                    }

                    if(lane == 0) ok = mbar_wait(smem_u32(s_full), n & 1u, abort_flag, 47);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if(!ok) break;
                    n++;
                    tcgen05_fence_after();

                    float v[kHalfKeys];
#pragma unroll
                    for(int j = 0; j < 4; j++) tmem_load_32_issue(lane_base + half * kHalfKeys + j * 32, v + j * 32);
                    tmem_load_wait();
#pragma unroll
                    for(int j = 0; j < 4; j++) tmem_load_pin_32(v + j * 32);
                    if(sweep == 0)
                    {
                        // the scores are in registers: the next tile's score MMAs may overwrite the accumulator
                        tcgen05_fence_before();
                        __syncwarp();
                        if(lane == 0) mbar_arrive(smem_u32(p_ready));
                    }

                    // log2-domain scores with the layer's masks, as in the single-tile kernel
                    float part_max[4] = { -INFINITY, -INFINITY, -INFINITY, -INFINITY };
#pragma unroll
                    for(int j = 0; j < 4; j++)
                    {
                        const int key0 = tile_key0 + j * 32;
                        const bool dead = key0 >= p.Sk || (p.causal && key0 > row0 + 31);
                        const bool special = pad_word[j] != 0 || key0 + 31 >= p.Sk || (p.causal && key0 + 31 > row0);
                        if(dead)
                        {
#pragma unroll
                            for(int i = 0; i < 32; i++) v[j * 32 + i] = -INFINITY;
                        }
                        else if(!special)
                        {
#pragma unroll
                            for(int i = 0; i < 32; i++) { v[j * 32 + i] *= to_log2; part_max[i & 3] = fmaxf(part_max[i & 3], v[j * 32 + i]); }
                        }
                        else
                        {
#pragma unroll
                            for(int i = 0; i < 32; i++)
                            {
                                const int key = key0 + i;
                                float t = v[j * 32 + i] * to_log2;
                                if((pad_word[j] >> i) & 1u) t = -1e9f * kLog2e;
                                if((p.causal && key > q_row) || key >= p.Sk) t = -INFINITY;
                                v[j * 32 + i] = t;
                                part_max[i & 3] = fmaxf(part_max[i & 3], t);
                            }
                        }
                    }

                    if(sweep == 0)
                    {
                        const float tile_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3]));
                        const float new_max = fmaxf(run_max, tile_max);
                        if(new_max > -INFINITY)
                        {
                            float part_sum[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
                            for(int i = 0; i < kHalfKeys; i++) part_sum[i & 3] += exp2_approx(v[i] - new_max);
                            run_sum = run_sum * exp2_approx(run_max - new_max) + ((part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]));
                            run_max = new_max;
                        }
                        if(kt == live - 1)
                        {
                            // the two halves of the row agree on its maximum and its sum
                            exchange[half * kQRows + r_local] = run_max;
                            pair_barrier(quadrant);
                            const float whole_max = fmaxf(run_max, exchange[(half ^ 1) * kQRows + r_local]);
                            pair_barrier(quadrant);
                            const float mine = run_max > -INFINITY ? run_sum * exp2_approx(run_max - whole_max) : 0.f;
                            exchange[half * kQRows + r_local] = mine;
                            pair_barrier(quadrant);
                            const float total = mine + exchange[(half ^ 1) * kQRows + r_local];
                            pair_barrier(quadrant);
                            row_max = whole_max > -INFINITY ? whole_max : 0.f;
                            inv = total > 0.f ? 1.0f / total : 0.f;
                        }
                    }
                    else
                    {
                        // exponentials against the row's final maximum, unnormalised and rounded to tf32 for the tensor core
#pragma unroll
                        for(int i = 0; i < kHalfKeys; i++) v[i] = round_tf32(exp2_approx(v[i] - row_max));
#pragma unroll
                        for(int j = 0; j < 4; j++) tmem_store_32_issue(lane_base + half * kHalfKeys + j * 32, v + j * 32);
                        tmem_store_wait();
                        tcgen05_fence_before();
                        __syncwarp();
                        if(lane == 0) mbar_arrive(smem_u32(p_ready));    // the context MMAs of this tile may start

                        // the normalised weights of this tile leave from the registers while those MMAs run
#pragma unroll
                        for(int j = 0; j < 4; j++)
                        {
                            const int block = kt * 8 + half * 4 + j;
                            if(block < p.key_blocks && row0 < p.Sq) stage_and_store(&map_p, warp_blocks, staged, v + j * 32, inv, lane, block * 32, row0, it.h, it.b);
                        }

                        if(kt == live - 1)
                        {
                            if(lane == 0) ok = mbar_wait(smem_u32(o_full), items_done & 1u, abort_flag, 48);
                            ok = __shfl_sync(0xffffffffu, ok, 0);
                            if(!ok) break;
                            tcgen05_fence_after();
#pragma unroll
                            for(int c = 0; c < KB; c++)
                            {
                                if((c & 1) != half) continue;    // the two warps of a quadrant take alternate 32-column blocks
                                float o[32];
                                __syncwarp();
                                tmem_load_32_issue(lane_base + O_COL + c * 32, o);
                                tmem_load_wait();
                                tmem_load_pin_32(o);
                                if(row0 < p.Sq) stage_and_store(&map_ctx, warp_blocks, staged, o, inv, lane, it.h * HD + c * 32, row0, 0, it.b);
                            }
                            tcgen05_fence_before();
                            __syncwarp();
                            if(lane == 0) mbar_arrive(smem_u32(o_free));
                        }
                    }
                }
            if(!ok) break;

            // key tiles the causal mask removes entirely: their weights are zeros
            if(live < p.key_tiles && row0 < p.Sq)
            {
                float zeros[32];
#pragma unroll
                for(int i = 0; i < 32; i++) zeros[i] = 0.f;
                for(int kt = live; kt < p.key_tiles; kt++)
                    for(int j = 0; j < 4; j++)
                    {
                        const int block = kt * 8 + half * 4 + j;
                        if(block < p.key_blocks) stage_and_store(&map_p, warp_blocks, staged, zeros, 1.0f, lane, block * 32, row0, it.h, it.b);
                    }
            }
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

// ---------------------------------------------------------------------------------------
// backward: map_q = dO, map_k = V (K-major), map_v = K (MN-major), map_p = dS (store), map_ctx = dQ (store),
// map_in = attention weights (load)
// ---------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_long_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_p,
                          const __grid_constant__ CUtensorMap map_ctx, const __grid_constant__ CUtensorMap map_in, const AttnParams p)
{
    static_assert(HD == 64, "one dQ block per softmax warp");
    constexpr int KB = HD / 32;
    constexpr int Q_BYTES = KB * kQRows * 128;
    constexpr int K_BYTES = KB * kMaxKeys * 128;
    constexpr int V_BYTES = KB * kMaxKeys * 128;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t O_COL = kMaxKeys;
    constexpr uint32_t IDESC_O = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(kQRows >> 4) << 24);
    constexpr int kRing = 4;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem;
    uint8_t* k_smem = q_smem + Q_BYTES;                      // V (K-major) for the dP MMAs, then K (MN-major) for the dQ MMAs
    uint8_t* v_smem = k_smem;
    uint8_t* stage_smem = k_smem + K_BYTES;
    float* exchange = reinterpret_cast<float*>(stage_smem + kSoftmaxWarps * kRing * kBlock);
    uint64_t* bars = reinterpret_cast<uint64_t*>(exchange + 2 * kQRows);
    uint64_t* qk_full = bars + 0;
    uint64_t* v_full = bars + 1;
    uint64_t* qk_empty = bars + 2;
    uint64_t* v_empty = bars + 3;
    uint64_t* s_full = bars + 4;
    uint64_t* p_ready = bars + 5;
    uint64_t* o_full = bars + 6;
    uint64_t* o_free = bars + 7;
    uint64_t* p_in = bars + 8;                              // [8 warps][4 blocks]: attention-weight blocks landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8 + 4 * kSoftmaxWarps);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if(threadIdx.x == 0)
    {
        mbar_init(smem_u32(qk_full), 1); mbar_init(smem_u32(v_full), 1);
        mbar_init(smem_u32(qk_empty), 1); mbar_init(smem_u32(v_empty), 1);
        mbar_init(smem_u32(s_full), 1); mbar_init(smem_u32(o_full), 1);
        mbar_init(smem_u32(p_ready), kSoftmaxWarps); mbar_init(smem_u32(o_free), kSoftmaxWarps);
        for(int i = 0; i < 4 * kSoftmaxWarps; i++) mbar_init(smem_u32(p_in + i), 1);
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
    pdl_wait();

    // one step per live key tile; n counts steps and gives the parity of every per-step barrier
    if(warp == 0)
    {
        if(lane == 0)
        {
            uint32_t n = 0;
            int qk_armed = -1, v_armed = -1;
            bool ok = true;
            for(long long w = blockIdx.x; ok && w < p.items; w += gridDim.x)
            {
                const AttnItem it = decode_item(p, w);
                const int live = live_key_tiles(p, it.q_tile);
                for(int kt = 0; kt < live; kt++, n++)
                {
                    // V takes the buffer the previous step's K was in, which that step's dQ MMAs read
                    if(!mbar_wait(smem_u32(v_empty), (n & 1u) ^ 1u, abort_flag, 51)) { ok = false; break; }
                    mbar_arrive_expect_tx(smem_u32(qk_full), (kt == 0 ? Q_BYTES : 0) + K_BYTES);
                    qk_armed = (int)(n & 1u);
#pragma unroll
                    for(int kb = 0; kb < KB; kb++)
                    {
                        if(kt == 0) tma_load_4d(smem_u32(q_smem + kb * kQRows * 128), &map_q, smem_u32(qk_full), it.h * HD + kb * 32, it.q_tile * kQRows, 0, it.b);
                        tma_load_4d(smem_u32(k_smem + kb * kMaxKeys * 128), &map_k, smem_u32(qk_full), it.h * HD + kb * 32, kt * kMaxKeys, 0, it.b);
                    }
                    // K takes the place of V as soon as THIS step's dP MMAs have read V
                    if(!mbar_wait(smem_u32(qk_empty), n & 1u, abort_flag, 52)) { ok = false; break; }
                    mbar_arrive_expect_tx(smem_u32(v_full), V_BYTES);
                    v_armed = (int)(n & 1u);
                    tma_load_5d(smem_u32(v_smem), &map_v, smem_u32(v_full), 0, kt * kMaxKeys, it.h * KB, 0, it.b);
                }
            }
            if(*abort_flag)
            {
                drain_phase(qk_full, qk_armed);
                drain_phase(v_full, v_armed);
            }
        }
    }
    else if(warp == 1)
    {
        if(lane == 0)
        {
            uint32_t n = 0, items_done = 0;
            bool ok = true;
            for(long long w = blockIdx.x; ok && w < p.items; w += gridDim.x, items_done++)
            {
                const AttnItem it = decode_item(p, w);
                const int live = live_key_tiles(p, it.q_tile);
                for(int kt = 0; kt < live; kt++, n++)
                {
                    const int keys = min(kMaxKeys, p.Sk - kt * kMaxKeys);
                    const int blocks = (keys + 31) / 32;
                    const uint32_t idesc_s = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)((blocks * 32) >> 3) << 17) | ((uint32_t)(kQRows >> 4) << 24);
                    if(!mbar_wait(smem_u32(qk_full), n & 1u, abort_flag, 53)) { ok = false; break; }
                    tcgen05_fence_after();
#pragma unroll
                    for(int kb = 0; kb < KB; kb++)
                    {
                        const uint64_t a_desc = make_smem_desc(smem_u32(q_smem + kb * kQRows * 128), 16, 1024, 2);
                        const uint64_t b_desc = make_smem_desc(smem_u32(k_smem + kb * kMaxKeys * 128), 16, 1024, 2);
#pragma unroll
                        for(int j = 0; j < 4; j++)
                            tcgen05_mma_tf32(tmem_base, a_desc + (uint64_t)(j * 32 >> 4), b_desc + (uint64_t)(j * 32 >> 4), idesc_s, (kb > 0 || j > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(smem_u32(qk_empty));           // V has been read: K may take its place
                    tcgen05_commit(smem_u32(s_full));             // dP complete

                    if(!mbar_wait(smem_u32(v_full), n & 1u, abort_flag, 54)) { ok = false; break; }
                    if(!mbar_wait(smem_u32(p_ready), n & 1u, abort_flag, 55)) { ok = false; break; }
                    if(kt == 0 && !mbar_wait(smem_u32(o_free), (items_done & 1u) ^ 1u, abort_flag, 56)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint64_t v_desc = make_smem_desc(smem_u32(v_smem), kMaxKeys * 128, 512, 1);
                    const int k_steps = blocks * 4;
                    for(int kk = 0; kk < k_steps; kk++)
                        tcgen05_mma_tf32_a_tmem(tmem_base + O_COL, tmem_base + (uint32_t)(kk * 8), v_desc + (uint64_t)(kk * 1024 >> 4), IDESC_O,
                                                (kt > 0 || kk > 0) ? 1u : 0u);
                    tcgen05_commit(smem_u32(v_empty));
                    if(kt == live - 1) tcgen05_commit(smem_u32(o_full));
                }
            }
        }
    }
    else
    {
        const int quadrant = warp & 3;
        const int half = (warp - 2) >> 2;
        const int r_local = quadrant * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quadrant * 32) << 16);
        const uint32_t warp_blocks = smem_u32(stage_smem + (warp - 2) * kRing * kBlock);
        uint64_t* my_in = p_in + (warp - 2) * 4;
        uint32_t in_phase[4] = { 0, 0, 0, 0 };
        uint32_t n = 0, items_done = 0;
        bool ok = true;
        for(long long w = blockIdx.x; ok && w < p.items; w += gridDim.x, items_done++)
        {
            const AttnItem it = decode_item(p, w);
            const int live = live_key_tiles(p, it.q_tile);
            const int row0 = it.q_tile * kQRows + quadrant * 32;
            const int q_row = row0 + lane;
            const bool rows_live = row0 < p.Sq;

            // delta = sum_d dO[row, d] * O[row, d]: the row sum of P * dP over all keys, taken without P
            constexpr int kPart = HD / 2;
            float delta = 0.f;
            if(q_row < p.Sq)
            {
                const long long at = ((long long)it.b * p.Sq + q_row) * p.E + it.h * HD + half * kPart;
#pragma unroll
                for(int c = 0; c < kPart / 4; c++)
                {
                    const float4 o = ld4(p.context + at + 4 * c), g = ld4(p.d_context + at + 4 * c);
                    delta += (o.x * g.x + o.y * g.y) + (o.z * g.z + o.w * g.w);
                }
            }

            for(int kt = 0; kt < live; kt++)
            {
                // this tile's four blocks of attention weights into the ring, once the copies that last read it have left
                if(lane == 0)
                {
                    bulk_wait_read_0();
                    for(int jb = 0; jb < 4; jb++)
                        if(rows_live && kt * 8 + half * 4 + jb < p.key_blocks)
                        {
                            mbar_arrive_expect_tx(smem_u32(my_in + jb), kBlock);
                            tma_load_4d(warp_blocks + jb * kBlock, &map_in, smem_u32(my_in + jb), (kt * 8 + half * 4 + jb) * 32, row0, it.h, it.b);
                        }
                }
                __syncwarp();

                if(lane == 0) ok = mbar_wait(smem_u32(s_full), n & 1u, abort_flag, 57);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if(!ok) break;
                n++;
                tcgen05_fence_after();

                if(kt == 0)
                {
                    exchange[half * kQRows + r_local] = delta;
                    pair_barrier(quadrant);
                    delta += exchange[(half ^ 1) * kQRows + r_local];
                    pair_barrier(quadrant);
                }

                // dS = P * (dP - delta), 32 columns at a time; its tf32-rounded copy goes back to tensor memory over dP
                float dp[2][32];
                tmem_load_32_issue(lane_base + half * kHalfKeys, dp[0]);
#pragma unroll
                for(int j = 0; j < 4; j++)
                {
                    const int block = kt * 8 + half * 4 + j;
                    const uint32_t buffer = warp_blocks + (uint32_t)j * kBlock;
                    const uint32_t bar = smem_u32(my_in + j);
                    float* d = dp[j & 1];
                    tmem_load_wait();
                    tmem_load_pin_32(d);
                    if(j + 1 < 4) tmem_load_32_issue(lane_base + half * kHalfKeys + (j + 1) * 32, dp[(j + 1) & 1]);
                    if(ok && rows_live && block < p.key_blocks)
                    {
                        if(lane == 0) ok = mbar_wait(bar, in_phase[j], abort_flag, 58);
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if(ok)
                        {
                            mbar_try_wait(bar, in_phase[j]);           // every lane observes the completed phase itself
                            in_phase[j] ^= 1;
                            float4 w4[8];
#pragma unroll
                            for(int q4 = 0; q4 < 8; q4++)
                            {
                                const uint32_t at = buffer + (uint32_t)lane * 128u + (uint32_t)((q4 ^ (lane & 7)) << 4);
                                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(w4[q4].x), "=f"(w4[q4].y), "=f"(w4[q4].z), "=f"(w4[q4].w) : "r"(at));
                            }
#pragma unroll
                            for(int q4 = 0; q4 < 8; q4++)
                            {
                                const uint32_t at = buffer + (uint32_t)lane * 128u + (uint32_t)((q4 ^ (lane & 7)) << 4);
                                const float d0 = w4[q4].x * (d[q4 * 4] - delta), d1 = w4[q4].y * (d[q4 * 4 + 1] - delta);
                                const float d2 = w4[q4].z * (d[q4 * 4 + 2] - delta), d3 = w4[q4].w * (d[q4 * 4 + 3] - delta);
                                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(at), "f"(d0), "f"(d1), "f"(d2), "f"(d3));
                                d[q4 * 4] = round_tf32(d0); d[q4 * 4 + 1] = round_tf32(d1);
                                d[q4 * 4 + 2] = round_tf32(d2); d[q4 * 4 + 3] = round_tf32(d3);
                            }
                            fence_async_shared();
                            __syncwarp();
                            if(lane == 0)
                            {
                                tma_store_4d(&map_p, buffer, block * 32, row0, it.h, it.b);
                                bulk_commit();
                            }
                            __syncwarp();
                        }
                    }
                    else
                    {
#pragma unroll
                        for(int i = 0; i < 32; i++) d[i] = 0.f;
                    }
                    tmem_store_32_issue(lane_base + half * kHalfKeys + j * 32, d);
                }
                if(!ok) break;
                tmem_store_wait();
                tcgen05_fence_before();
                __syncwarp();
                if(lane == 0) mbar_arrive(smem_u32(p_ready));    // the dQ MMAs of this tile may start
            }
            if(!ok) break;

            // dQ = scale * (sum over the key tiles of dS K): this warp's 32 x 32 block, staged in ring block 3
            if(lane == 0) ok = mbar_wait(smem_u32(o_full), items_done & 1u, abort_flag, 59);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if(!ok) break;
            tcgen05_fence_after();
            {
                const int c = half;
                const uint32_t buffer = warp_blocks + 3 * kBlock;
                float o[32];
                tmem_load_32_issue(lane_base + O_COL + c * 32, o);
                tmem_load_wait();
                tmem_load_pin_32(o);
                tcgen05_fence_before();
                __syncwarp();
                if(lane == 0) mbar_arrive(smem_u32(o_free));     // the accumulator may take the next item's dQ
                if(rows_live)
                {
                    if(lane == 0) bulk_wait_read_0();            // the last tile's dS copy has left ring block 3
                    __syncwarp();
#pragma unroll
                    for(int q4 = 0; q4 < 8; q4++)
                    {
                        const uint32_t dst = buffer + (uint32_t)lane * 128u + (uint32_t)((q4 ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(dst), "f"(o[q4 * 4] * p.scale), "f"(o[q4 * 4 + 1] * p.scale),
                                     "f"(o[q4 * 4 + 2] * p.scale), "f"(o[q4 * 4 + 3] * p.scale));
                    }
                    __syncwarp();
                    if(p.d_bias_q)
                    {
                        // lane L adds up column L of the staged block (rows past Sq hold zeros) for the query-bias gradient
                        float part[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
                        for(int r = 0; r < 32; r++)
                        {
                            const uint32_t at = buffer + (uint32_t)r * 128u + (uint32_t)(((lane >> 2) ^ (r & 7)) << 4) + (uint32_t)(lane & 3) * 4u;
                            float x;
                            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x) : "r"(at));
                            part[r & 3] += x;
                        }
                        atomicAdd(p.d_bias_q + it.h * HD + c * 32 + lane, (part[0] + part[1]) + (part[2] + part[3]));
                    }
                    fence_async_shared();
                    __syncwarp();
                    if(lane == 0) { tma_store_4d(&map_ctx, buffer, it.h * HD + c * 32, row0, 0, it.b); bulk_commit(); }
                    __syncwarp();
                }
            }

            // key tiles the causal mask removes entirely: their score gradient is zero
            if(live < p.key_tiles && rows_live)
            {
                const uint32_t buffer = warp_blocks;             // ring block 0, filled with zeros once its last copy has left
                if(lane == 0) bulk_wait_read_0();
                __syncwarp();
#pragma unroll
                for(int q4 = 0; q4 < 8; q4++)
                    asm volatile("st.shared.v4.f32 [%0], {%1, %1, %1, %1};" :: "r"(buffer + (uint32_t)lane * 128u + (uint32_t)(q4 << 4)), "f"(0.f));
                fence_async_shared();
                __syncwarp();
                if(lane == 0)
                {
                    for(int kt = live; kt < p.key_tiles; kt++)
                        for(int j = 0; j < 4; j++)
                        {
                            const int block = kt * 8 + half * 4 + j;
                            if(block < p.key_blocks) tma_store_4d(&map_p, buffer, block * 32, row0, it.h, it.b);
                        }
                    bulk_commit();
                }
                __syncwarp();
            }
        }
        if(lane == 0) bulk_wait_all();
    }

    tcgen05_fence_before();
    __syncthreads();
    if(warp == 1)
    {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

static AttnParams long_params(long long B, long long Sq, long long Sk, long long E, long long H, float scale)
{
    AttnParams p = {};
    p.B = (int)B; p.H = (int)H; p.Sq = (int)Sq; p.Sk = (int)Sk;
    p.q_tiles = (int)((Sq + kQRows - 1) / kQRows);
    p.key_blocks = (int)((Sk + 31) / 32);
    p.key_tiles = (int)((Sk + kMaxKeys - 1) / kMaxKeys);
    p.scale = scale;
    p.items = B * H * p.q_tiles;
    p.E = E;
    return p;
}

}  // namespace tc

bool attention_long_supported(long long B, long long Sq, long long Sk, long long E, long long H)
{
    if(H <= 0 || E % H != 0 || E / H != 64) return false;
    if(Sk <= tc::kMaxKeys || (Sk & 3) != 0 || Sk >= (1LL << 24)) return false;
    if(B >= 65536 || Sq >= (1LL << 24)) return false;
    return tc::encode_tiled() != nullptr;
}

int attention_long_fwd_launch(const float* q, const float* k, const float* v, const unsigned char* key_is_pad,
                              float* weights, float* context, long long B, long long Sq, long long Sk, long long E, long long H,
                              int causal, float scale, cudaStream_t stream)
{
    using namespace tc;
    constexpr int HD = 64;
    AttnParams p = long_params(B, Sq, Sk, E, H, scale);
    p.key_is_pad = key_is_pad;
    p.causal = causal;

    CUtensorMap map_q, map_k, map_v, map_p, map_ctx;
    bool ok = make_map(&map_q, q, E, Sq, E, 1, 0, (int)B, Sq * E, 32, kQRows, false);
    ok = ok && make_map(&map_k, k, E, Sk, E, 1, 0, (int)B, Sk * E, 32, kMaxKeys, false);
    ok = ok && make_wide_map(&map_v, v, E, Sk, E, 1, 0, (int)B, Sk * E, HD / 32, kMaxKeys);
    ok = ok && make_map(&map_p, weights, Sk, Sq, Sk, (int)H, Sq * Sk, (int)B, H * Sq * Sk, 32, 32, false, false);
    ok = ok && make_map(&map_ctx, context, E, Sq, E, 1, 0, (int)B, Sq * E, 32, 32, false, false);
    if(!ok) return ONN_ERR_UNSUPPORTED;
    static PerDeviceBytes configured;
    if(!ensure_dynamic_smem(attention_long_fwd_kernel<HD>, configured, kLongSmem)) return ONN_ERR_CUDA;
    const int grid = (int)(p.items < sm_limit() ? p.items : sm_limit());
    const cudaError_t launched = launch_overlapped(attention_long_fwd_kernel<HD>, dim3(grid), dim3(kAttnThreads), kLongSmem, stream,
                                                   map_q, map_k, map_v, map_p, map_ctx, p);
    count_launch();
    return launched == cudaSuccess ? launch_status() : ONN_ERR_CUDA;
}

int attention_long_bwd_launch(const float* k, const float* v, const float* weights, const float* context, const float* d_context,
                              float* d_scores, float* d_q, float* d_bias_q, long long B, long long Sq, long long Sk, long long E, long long H,
                              int causal, float scale, cudaStream_t stream)
{
    using namespace tc;
    constexpr int HD = 64;
    AttnParams p = long_params(B, Sq, Sk, E, H, scale);
    p.causal = causal;                                       // only to skip the key tiles whose weights are all zero
    p.context = context;
    p.d_context = d_context;
    p.d_bias_q = d_bias_q;

    CUtensorMap map_do, map_v, map_k, map_ds, map_dq, map_w;
    bool ok = make_map(&map_do, d_context, E, Sq, E, 1, 0, (int)B, Sq * E, 32, kQRows, false);
    ok = ok && make_map(&map_v, v, E, Sk, E, 1, 0, (int)B, Sk * E, 32, kMaxKeys, false);
    ok = ok && make_wide_map(&map_k, k, E, Sk, E, 1, 0, (int)B, Sk * E, HD / 32, kMaxKeys);
    ok = ok && make_map(&map_ds, d_scores, Sk, Sq, Sk, (int)H, Sq * Sk, (int)B, H * Sq * Sk, 32, 32, false, false);
    ok = ok && make_map(&map_dq, d_q, E, Sq, E, 1, 0, (int)B, Sq * E, 32, 32, false, false);
    ok = ok && make_map(&map_w, weights, Sk, Sq, Sk, (int)H, Sq * Sk, (int)B, H * Sq * Sk, 32, 32, false, false);
    if(!ok) return ONN_ERR_UNSUPPORTED;
    static PerDeviceBytes configured;
    if(!ensure_dynamic_smem(attention_long_bwd_kernel<HD>, configured, kLongSmem)) return ONN_ERR_CUDA;
    const int grid = (int)(p.items < sm_limit() ? p.items : sm_limit());
    const cudaError_t launched = launch_overlapped(attention_long_bwd_kernel<HD>, dim3(grid), dim3(kAttnThreads), kLongSmem, stream,
                                                   map_do, map_v, map_k, map_ds, map_dq, map_w, p);
    count_launch();
    return launched == cudaSuccess ? launch_status() : ONN_ERR_CUDA;
}

const unsigned int* attention_long_status_word() { return tc::status_word_address(); }

int attention_long_read_status()
{
    unsigned int status = 0;
    if(tc::read_and_clear_status(&status) != 0) return ONN_ERR_CUDA;
    return status == 0 ? ONN_OK : ONN_ERR_DEVICE_TIMEOUT;
}

}  // namespace onn
