// Attention core on the Blackwell tensor cores: scores, masks, softmax and context in ONE kernel.
//
// For one (batch, head, 128-query tile) a CTA computes
//     S = Q K^T (tcgen05.mma, kind::tf32, accumulator in tensor memory, 128 lanes x up to 256 columns)
//     P = softmax(scale * S with the key-padding and causal masks)
//     O = P V   (second MMA: A operand read straight from tensor memory, V from shared memory)
// and writes P (the attention weights the layer keeps for back-propagation) and O (its head's column
// slice of the concatenated context) once.  The score matrix never makes the round trips through HBM
// that separate GEMM / softmax / GEMM launches need: traffic per (batch, head) drops from ~7 passes
// over the [Sq, Sk] matrix to the single write of P.
//
// Shapes: head size 64, source length <= 256 (one accumulator holds a whole row of scores), any query
// length (tiles of 128 rows, ragged tiles are zero-filled on load and clipped on store by the copy engine).
// The layer front end falls back to the separate kernels for anything else.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer (owns tensor memory), warps 2..9 = softmax and
// output.  A warp may read only the 32 accumulator lanes (query rows) its id selects, so warps w and
// w + 4 share a quadrant and split its columns: each thread holds 128 scores of one row in registers
// from ONE tensor-memory load (a round trip costs ~500 cycles, so the row is never re-read), the two
// halves exchange row maximum and row sum through shared memory, the unnormalised exponentials go
// back to tensor memory (rounded to tf32) for the context MMA, and the normalised weights leave from
// the registers through swizzled staging blocks and TMA stores while that MMA runs.
// CTAs are persistent: the producer fetches the next item's Q/K as soon as the score MMAs have read the
// current ones, V as soon as the context MMAs have, and the next item's scores are computed while this
// item's weights are still being written.  All barrier waits are bounded (tcgen05.cuh).
#include <cmath>
#include <cstdlib>

#include "attention_internal.h"
#include "attention_parts.cuh"
#include "common.cuh"
#include "launch_counter.h"
#include "tcgen05.cuh"
#include "work_ring.cuh"

namespace onn
{
namespace tc
{

// BACKWARD = false: map_q = Q, map_k = K (K-major), map_v = V (MN-major), map_p = attention weights (store),
//                   map_ctx = context (store).
// BACKWARD = true : the same two MMAs compute dP = dO V^T and dQ = dS K, so map_q = dO, map_k = V (K-major),
//                   map_v = K (MN-major), map_p = dS (store), map_ctx = dQ (store), map_in = attention weights (load).
template <int HD, bool BACKWARD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_core_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_p,
                      const __grid_constant__ CUtensorMap map_ctx, const __grid_constant__ CUtensorMap map_in, const AttnParams p)
{
    constexpr int KB = HD / 32;                             // 32-float k-blocks of the head dimension
    constexpr int Q_BYTES = KB * kQRows * 128;              // K-major [128 rows][32 floats] per k-block
    constexpr int K_BYTES = KB * kMaxKeys * 128;            // K-major [256 rows][32 floats] per k-block
    constexpr int V_BYTES = KB * kMaxKeys * 128;            // MN-major [HD / 32 atoms][256 key rows][32 floats]
    constexpr uint32_t TMEM_COLS = 512;                     // scores 0..255, context 256..256+HD
    constexpr uint32_t O_COL = kMaxKeys;
    // D = fp32, A = B = tf32; context MMA: A from tensor memory (K-major), B = V MN-major, N = HD
    constexpr uint32_t IDESC_O = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(kQRows >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_smem = smem;
    uint8_t* k_smem = q_smem + Q_BYTES;
    // forward: V has its own 64 KiB and every softmax warp two staging blocks; backward: the second MMA's operand
    // (K, MN-major) follows the first one's (V, K-major) in the SAME 64 KiB, which pays for four ring blocks per warp
    constexpr int kRing = BACKWARD ? 4 : 2;
    uint8_t* v_smem = BACKWARD ? k_smem : k_smem + K_BYTES;
    uint8_t* stage_smem = BACKWARD ? k_smem + K_BYTES : v_smem + V_BYTES;
    float* exchange = reinterpret_cast<float*>(stage_smem + kSoftmaxWarps * kRing * kBlock);     // [2 halves][128 rows]
    uint64_t* bars = reinterpret_cast<uint64_t*>(exchange + 2 * kQRows);
    uint64_t* qk_full = bars + 0;
    uint64_t* v_full = bars + 1;
    uint64_t* qk_empty = bars + 2;
    uint64_t* v_empty = bars + 3;
    uint64_t* s_full = bars + 4;
    uint64_t* p_ready = bars + 5;
    uint64_t* o_full = bars + 6;
    uint64_t* o_free = bars + 7;
    uint64_t* p_in = bars + 8;                              // [8 warps][4 blocks]: attention-weight blocks landed (backward)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8 + 4 * kSoftmaxWarps);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    WorkRing* ring = reinterpret_cast<WorkRing*>(bars + 8 + 4 * kSoftmaxWarps + 1);   // producer -> MMA issuer and softmax warps
    static_assert((8 + 4 * kSoftmaxWarps + 1) * 8 + sizeof(WorkRing) <= 512, "barriers beyond their 512 bytes");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if(threadIdx.x == 0)
    {
        mbar_init(smem_u32(qk_full), 1); mbar_init(smem_u32(v_full), 1);
        mbar_init(smem_u32(qk_empty), 1); mbar_init(smem_u32(v_empty), 1);
        mbar_init(smem_u32(s_full), 1); mbar_init(smem_u32(o_full), 1);
        mbar_init(smem_u32(p_ready), kSoftmaxWarps); mbar_init(smem_u32(o_free), kSoftmaxWarps);
        for(int i = 0; i < 4 * kSoftmaxWarps; i++) mbar_init(smem_u32(p_in + i), 1);
        work_ring_init(ring, 1 + kSoftmaxWarps);
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
    // Only now may the counter be touched: a counter of the pool can come round to two launches that follow each other
    // on the stream (one of them replayed from a graph captured long ago), and before the wait the earlier one may
    // still be running.
    const WorkSource source = { p.work_counter, (uint32_t)p.items, gridDim.x };
    const WorkView work = { ring, p.work_counter != nullptr, (uint32_t)p.items };
    uint32_t first_work = kNoWork;
    if(threadIdx.x == 0) first_work = source.fetch(0, blockIdx.x, gridDim.x);

    if(warp == 0)
    {
        // ---------------- TMA producer ----------------
        if(lane == 0)
        {
            // The producer is also the scheduler.  It asks for item t + 1 before it copies item t (the counter's round
            // trip runs under the copies) and tells the other roles once those copies are on their way, so nobody holds
            // more than one item beyond the one it is working on.
            uint32_t ph = 0;
            uint32_t w = first_work;
            bool told = work.publish(0, w, abort_flag, 20);
            for(uint32_t turn = 0; told && w != kNoWork; turn++, ph ^= 1)
            {
                const uint32_t ahead = source.fetch(turn + 1, blockIdx.x, gridDim.x);
                const AttnItem it = decode_item(p, w);
                // forward: Q and K may be replaced once the previous item's score MMAs have read them; backward: V shares
                // its buffer with the previous item's K, which the previous item's second group of MMAs reads
                if(!mbar_wait(smem_u32(BACKWARD ? v_empty : qk_empty), ph ^ 1, abort_flag, 21)) break;
                mbar_arrive_expect_tx(smem_u32(qk_full), Q_BYTES + K_BYTES);
#pragma unroll
                for(int kb = 0; kb < KB; kb++)
                {
                    tma_load_4d(smem_u32(q_smem + kb * kQRows * 128), &map_q, smem_u32(qk_full), it.h * HD + kb * 32, it.q_tile * kQRows, 0, it.b);
                    tma_load_4d(smem_u32(k_smem + kb * kMaxKeys * 128), &map_k, smem_u32(qk_full), it.h * HD + kb * 32, 0, 0, it.b);
                }
                // forward: V's buffer is free once the previous item's context MMAs are done; backward: K takes the
                // place of V as soon as THIS item's first group of MMAs has read V
                if(!mbar_wait(smem_u32(BACKWARD ? qk_empty : v_empty), BACKWARD ? ph : ph ^ 1, abort_flag, 22)) break;
                mbar_arrive_expect_tx(smem_u32(v_full), V_BYTES);
                tma_load_5d(smem_u32(v_smem), &map_v, smem_u32(v_full), 0, 0, it.h * KB, 0, it.b);
                w = ahead;
                told = work.publish(turn + 1, w, abort_flag, 20);
            }
            if(*abort_flag)
            {
                const unsigned long long start = clock64();
                while(clock64() - start < 200000ull) { }    // let copies in flight land before shared memory goes away
            }
        }
    }
    else if(warp == 1)
    {
        // ---------------- MMA issuer ----------------
        if(lane == 0)
        {
            const uint32_t idesc_s = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)((p.key_blocks * 32) >> 3) << 17) | ((uint32_t)(kQRows >> 4) << 24);
            uint32_t ph = 0;
            for(uint32_t turn = 0; work.take(turn, abort_flag, 24) != kNoWork; turn++, ph ^= 1)
            {
                // scores: the previous item's context MMAs were issued before these and the tensor pipe runs in order,
                // and every softmax thread had its scores in registers before those MMAs were released (p_ready)
                if(!mbar_wait(smem_u32(qk_full), ph, abort_flag, 23)) break;
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

                if(!mbar_wait(smem_u32(v_full), ph, abort_flag, 25)) break;
                if(!mbar_wait(smem_u32(p_ready), ph, abort_flag, 26)) break;
                if(!mbar_wait(smem_u32(o_free), ph ^ 1, abort_flag, 27)) break;
                tcgen05_fence_after();
                const uint64_t v_desc = make_smem_desc(smem_u32(v_smem), kMaxKeys * 128, 512, 1);
                const int k_steps = p.key_blocks * 4;        // 8 keys per MMA
                for(int kk = 0; kk < k_steps; kk++)
                    tcgen05_mma_tf32_a_tmem(tmem_base + O_COL, tmem_base + (uint32_t)(kk * 8), v_desc + (uint64_t)(kk * 1024 >> 4), IDESC_O, kk > 0 ? 1u : 0u);
                tcgen05_commit(smem_u32(v_empty));
                tcgen05_commit(smem_u32(o_full));
            }
        }
    }
    else
    {
        // ---------------- softmax and output (warps 2..9) ----------------
        const int quadrant = warp & 3;                       // accumulator lanes 32 * quadrant .. + 31
        const int half = (warp - 2) >> 2;                    // 0: key columns 0..127, 1: 128..255
        const int r_local = quadrant * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quadrant * 32) << 16);
        const uint32_t warp_blocks = smem_u32(stage_smem + (warp - 2) * kRing * kBlock);
        const float to_log2 = p.scale * kLog2e;
        unsigned int staged = 0;
        uint32_t in_phase[4] = { 0, 0, 0, 0 };
        if constexpr(BACKWARD)
        {
            // the first item's four blocks of attention weights
            const uint32_t first_item = lane == 0 ? work.peek(0, abort_flag, 31) : kNoWork;
            if(lane == 0 && first_item != kNoWork)
            {
                const AttnItem first = decode_item(p, first_item);
                const int first_row0 = first.q_tile * kQRows + quadrant * 32;
                for(int jb = 0; jb < 4; jb++)
                    if(first_row0 < p.Sq && half * 4 + jb < p.key_blocks)
                    {
                        mbar_arrive_expect_tx(smem_u32(p_in + (warp - 2) * 4 + jb), kBlock);
                        tma_load_4d(warp_blocks + jb * kBlock, &map_in, smem_u32(p_in + (warp - 2) * 4 + jb), (half * 4 + jb) * 32, first_row0, first.h, first.b);
                    }
            }
            __syncwarp();
        }
        uint32_t ph = 0;
        // The item of a turn is taken at the top of the turn.  The backward kernel also looks at the NEXT turn's item in
        // the middle of this one (it asks for that item's attention weights there) without taking it; nothing is
        // carried round the loop: the forward kernel in particular has no register to spare.
        for(uint32_t turn = 0; ; turn++, ph ^= 1)
        {
            const uint32_t w = work.warp_take(turn, lane, abort_flag, 32);
            if(w == kNoWork) break;
            const AttnItem it = decode_item(p, w);
            const int row0 = it.q_tile * kQRows + quadrant * 32;      // first query row of this warp
            const int q_row = row0 + lane;

            if constexpr(BACKWARD)
            {
                static_assert(!BACKWARD || HD == 64, "one dQ block per softmax warp");
                const bool rows_live = row0 < p.Sq;
                uint64_t* my_in = p_in + (warp - 2) * 4;

                // this thread's share of delta = sum_d dO[row, d] * O[row, d]: the row sum of P * dP, taken without P
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

                bool ok = true;
                if(lane == 0) ok = mbar_wait(smem_u32(s_full), ph, abort_flag, 28);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if(!ok) break;
                tcgen05_fence_after();

                exchange[half * kQRows + r_local] = delta;
                pair_barrier(quadrant);
                delta += exchange[(half ^ 1) * kQRows + r_local];
                if(p.delta_out && half == 0 && q_row < p.Sq) p.delta_out[((long long)it.b * p.H + it.h) * p.Sq + q_row] = delta;

                // dS = P * (dP - delta), 32 columns at a time.  dP comes from tensor memory one block ahead of its use; the
                // weights arrived in this warp's four ring blocks by TMA (requested while the previous item was still being
                // worked on); dS is formed in place in the ring block and leaves from there, and its tf32-rounded copy goes
                // back to tensor memory, over dP, as the A operand of the dQ MMA.
                float dp[2][32];
                tmem_load_32_issue(lane_base + half * kHalfKeys, dp[0]);
#pragma unroll
                for(int j = 0; j < 4; j++)
                {
                    const int block = half * 4 + j;
                    const uint32_t buffer = warp_blocks + (uint32_t)j * kBlock;
                    const uint32_t bar = smem_u32(my_in + j);
                    float* d = dp[j & 1];
                    tmem_load_wait();
                    tmem_load_pin_32(d);
                    if(j + 1 < 4) tmem_load_32_issue(lane_base + half * kHalfKeys + (j + 1) * 32, dp[(j + 1) & 1]);
                    if(ok && rows_live && block < p.key_blocks)
                    {
                        if(lane == 0) ok = mbar_wait(bar, in_phase[j], abort_flag, 30);
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
                            if(lane == 0 && !p.skip_score_gradient_store)
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
                if(lane == 0) mbar_arrive(smem_u32(p_ready));    // the dQ MMAs may start

                // the next item's weights take ring blocks 0..2 as soon as this item's copies have left them (block 3 stages dQ first)
                const uint32_t w_next = work.warp_peek(turn + 1, lane, abort_flag, 33);
                AttnItem next = it;
                int next_row0 = 0;
                bool next_live = false;
                if(w_next != kNoWork)
                {
                    next = decode_item(p, w_next);
                    next_row0 = next.q_tile * kQRows + quadrant * 32;
                    next_live = next_row0 < p.Sq;
                }
                if(lane == 0)
                {
                    bulk_wait_read_0();
                    for(int jb = 0; jb < 3; jb++)
                        if(next_live && half * 4 + jb < p.key_blocks)
                        {
                            mbar_arrive_expect_tx(smem_u32(my_in + jb), kBlock);
                            tma_load_4d(warp_blocks + jb * kBlock, &map_in, smem_u32(my_in + jb), (half * 4 + jb) * 32, next_row0, next.h, next.b);
                        }
                }
                __syncwarp();

                if(lane == 0) ok = mbar_wait(smem_u32(o_full), ph, abort_flag, 29);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if(!ok) break;
                tcgen05_fence_after();
                {
                    // dQ = scale * dS K: this warp's 32 x 32 block (columns 32 * half ..), staged in ring block 3
                    const int c = half;
                    const uint32_t buffer = warp_blocks + 3 * kBlock;
                    float o[32];
                    tmem_load_32_issue(lane_base + O_COL + c * 32, o);
                    tmem_load_wait();
                    tmem_load_pin_32(o);
                    if(rows_live)
                    {
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
                    }
                    if(lane == 0)
                    {
                        bulk_wait_read_0();
                        if(next_live && half * 4 + 3 < p.key_blocks)
                        {
                            mbar_arrive_expect_tx(smem_u32(my_in + 3), kBlock);
                            tma_load_4d(buffer, &map_in, smem_u32(my_in + 3), (half * 4 + 3) * 32, next_row0, next.h, next.b);
                        }
                    }
                    __syncwarp();
                }
            }
            else
            {
                // key-padding flags of this thread's four 32-key blocks, one word per block (the same in every lane)
                uint32_t pad_word[4];
#pragma unroll
                for(int j = 0; j < 4; j++)
                {
                    const int key = half * kHalfKeys + j * 32 + lane;
                    const bool flag = p.key_is_pad && key < p.Sk && p.key_is_pad[(long long)it.b * p.Sk + key] != 0;
                    pad_word[j] = __ballot_sync(0xffffffffu, flag);
                }

                bool ok = true;
                if(lane == 0) ok = mbar_wait(smem_u32(s_full), ph, abort_flag, 28);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if(!ok) break;
                tcgen05_fence_after();

                // this thread's 128 scores, one round trip
                float v[kHalfKeys];
#pragma unroll
                for(int j = 0; j < 4; j++) tmem_load_32_issue(lane_base + half * kHalfKeys + j * 32, v + j * 32);
                tmem_load_wait();
#pragma unroll
                for(int j = 0; j < 4; j++) tmem_load_pin_32(v + j * 32);

                // scores in the log2 domain with the layer's masks: padded keys are OVERWRITTEN with -1e9, keys after the
                // query (causal) and keys past the source length drop out; blocks that need no per-element test take the short path
                float part_max[4] = { -INFINITY, -INFINITY, -INFINITY, -INFINITY };   // four chains instead of one long one
#pragma unroll
                for(int j = 0; j < 4; j++)
                {
                    const int key0 = half * kHalfKeys + j * 32;
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
                float row_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3]));
                exchange[half * kQRows + r_local] = row_max;
                pair_barrier(quadrant);
                row_max = fmaxf(row_max, exchange[(half ^ 1) * kQRows + r_local]);
                pair_barrier(quadrant);                          // both have read: the slots may be rewritten

                // exponentials, unnormalised and rounded to tf32 for the tensor core
                float part_sum[4] = { 0.f, 0.f, 0.f, 0.f };
#pragma unroll
                for(int i = 0; i < kHalfKeys; i++)
                {
                    const float e = round_tf32(exp2_approx(v[i] - row_max));
                    part_sum[i & 3] += e;
                    v[i] = e;
                }
                float total = (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
#pragma unroll
                for(int j = 0; j < 4; j++) tmem_store_32_issue(lane_base + half * kHalfKeys + j * 32, v + j * 32);
                tmem_store_wait();
                tcgen05_fence_before();
                __syncwarp();
                if(lane == 0) mbar_arrive(smem_u32(p_ready));    // the context MMAs may start

                exchange[half * kQRows + r_local] = total;
                pair_barrier(quadrant);
                total += exchange[(half ^ 1) * kQRows + r_local];
                const float inv = total > 0.f ? 1.0f / total : 0.f;
                if(p.row_max_out && half == 0 && q_row < p.Sq)
                {
                    // what the key / value gradient kernel needs to form this row's weights again without reading them
                    const long long at = ((long long)it.b * p.H + it.h) * p.Sq + q_row;
                    p.row_max_out[at] = row_max;
                    p.row_inv_out[at] = inv;
                }

                // the attention weights leave from the registers while the context MMAs run
#pragma unroll
                for(int j = 0; j < 4; j++)
                {
                    const int block = half * 4 + j;
                    if(block < p.key_blocks && row0 < p.Sq) stage_and_store(&map_p, warp_blocks, staged, v + j * 32, inv, lane, block * 32, row0, it.h, it.b);
                }

                if(lane == 0) ok = mbar_wait(smem_u32(o_full), ph, abort_flag, 29);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if(!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for(int c = 0; c < KB; c++)
                {
                    if((c & 1) != half) continue;                // the two warps of a quadrant take alternate 32-column blocks
                    float o[32];
                    __syncwarp();
                    tmem_load_32_issue(lane_base + O_COL + c * 32, o);
                    tmem_load_wait();
                    tmem_load_pin_32(o);
                    if(row0 < p.Sq) stage_and_store(&map_ctx, warp_blocks, staged, o, inv, lane, it.h * HD + c * 32, row0, 0, it.b);
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if(lane == 0) mbar_arrive(smem_u32(o_free));
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

}  // namespace tc

static bool attention_shapes_supported(long long B, long long Sq, long long Sk, long long E, long long H)
{
    if(H <= 0 || E % H != 0 || E / H != 64) return false;
    if(Sk > tc::kMaxKeys || (Sk & 3) != 0) return false;              // one accumulator row; 16-byte pitch of the weights
    if(B >= 65536 || Sq >= (1LL << 30)) return false;
    return tc::encode_tiled() != nullptr;
}

bool attention_fwd_fused_supported(const float* q, const float* k, const float* v, const float* weights, const float* context,
                                   long long B, long long Sq, long long Sk, long long E, long long H)
{
    if(!host_aligned16(q) || !host_aligned16(k) || !host_aligned16(v) || !host_aligned16(weights) || !host_aligned16(context)) return false;
    return attention_shapes_supported(B, Sq, Sk, E, H);
}

bool attention_bwd_fused_supported(const float* k, const float* v, const float* weights, const float* context, const float* d_context,
                                   const float* d_scores, const float* d_q, long long B, long long Sq, long long Sk, long long E, long long H)
{
    if(!host_aligned16(k) || !host_aligned16(v) || !host_aligned16(weights) || !host_aligned16(context) || !host_aligned16(d_context) ||
       !host_aligned16(d_scores) || !host_aligned16(d_q)) return false;
    return attention_shapes_supported(B, Sq, Sk, E, H);
}

namespace tc
{
constexpr int kAttnHeadSize = 64;
// operands, ring / staging blocks, exchange array, alignment slack, barriers
constexpr int kAttnSmem = (kAttnHeadSize / 32) * (kQRows + 2 * kMaxKeys) * 128 + kSoftmaxWarps * 2 * kBlock + 2 * kQRows * 4 + 1024 + 512;
static_assert(kAttnSmem <= 232448, "beyond the shared memory of one CTA");

static AttnParams attention_params(long long B, long long Sq, long long Sk, long long E, long long H, float scale)
{
    AttnParams p = {};
    p.B = (int)B; p.H = (int)H; p.Sq = (int)Sq; p.Sk = (int)Sk;
    p.q_tiles = (int)((Sq + kQRows - 1) / kQRows);
    p.key_blocks = (int)((Sk + 31) / 32);
    p.scale = scale;
    p.items = B * H * p.q_tiles;
    p.E = E;
    return p;
}

template <bool BACKWARD>
static int launch_attention_core(const CUtensorMap& a, const CUtensorMap& b1, const CUtensorMap& b2, const CUtensorMap& w, const CUtensorMap& o,
                                 const CUtensorMap& in, const AttnParams& p, cudaStream_t stream)
{
    static PerDeviceBytes configured;                        // per instantiation and per device
    if(!ensure_dynamic_smem(attention_core_kernel<kAttnHeadSize, BACKWARD>, configured, kAttnSmem)) return ONN_ERR_CUDA;
    if(p.items >= (1LL << 31)) return ONN_ERR_UNSUPPORTED;
    const int grid = (int)(p.items < sm_limit() ? p.items : sm_limit());
    AttnParams launch_params = p;
    launch_params.work_counter = next_work_counter();       // items in the order the CTAs ask for them (null: fixed shares)
    const cudaError_t launched = launch_overlapped(attention_core_kernel<kAttnHeadSize, BACKWARD>, dim3(grid), dim3(kAttnThreads), kAttnSmem, stream, a, b1, b2, w, o, in,
                                                   launch_params);
    count_launch();
    return launched == cudaSuccess ? launch_status() : ONN_ERR_CUDA;
}
}  // namespace tc

int attention_fwd_fused_launch(const float* q, const float* k, const float* v, const unsigned char* key_is_pad,
                               float* weights, float* context, float* row_max_out, float* row_inv_out,
                               long long B, long long Sq, long long Sk, long long E, long long H,
                               int causal, float scale, cudaStream_t stream)
{
    using namespace tc;
    constexpr int HD = kAttnHeadSize;
    AttnParams p = attention_params(B, Sq, Sk, E, H, scale);
    p.key_is_pad = key_is_pad;
    p.causal = causal;
    p.row_max_out = row_max_out && row_inv_out ? row_max_out : nullptr;
    p.row_inv_out = row_inv_out;

    CUtensorMap map_q, map_k, map_v, map_p, map_ctx;
    bool ok = make_map(&map_q, q, E, Sq, E, 1, 0, (int)B, Sq * E, 32, kQRows, false);
    ok = ok && make_map(&map_k, k, E, Sk, E, 1, 0, (int)B, Sk * E, 32, kMaxKeys, false);
    ok = ok && make_wide_map(&map_v, v, E, Sk, E, 1, 0, (int)B, Sk * E, HD / 32, kMaxKeys);
    ok = ok && make_map(&map_p, weights, Sk, Sq, Sk, (int)H, Sq * Sk, (int)B, H * Sq * Sk, 32, 32, false, false);
    ok = ok && make_map(&map_ctx, context, E, Sq, E, 1, 0, (int)B, Sq * E, 32, 32, false, false);
    if(!ok) return ONN_ERR_UNSUPPORTED;
    return launch_attention_core<false>(map_q, map_k, map_v, map_p, map_ctx, map_p, p, stream);
}

// dS = P * (dP - rowsum(P * dP)) with dP = dO V^T, written to d_scores ([B, H, Sq, Sk]); dQ = scale * dS K written to
// d_q ([B, Sq, E]); the column sums of dQ are added to d_bias_q ([E], may be null).
int attention_bwd_fused_launch(const float* k, const float* v, const float* weights, const float* context, const float* d_context,
                               float* d_scores, float* d_q, float* d_bias_q, float* delta_out, int store_score_gradient,
                               long long B, long long Sq, long long Sk, long long E, long long H,
                               float scale, cudaStream_t stream)
{
    using namespace tc;
    constexpr int HD = kAttnHeadSize;
    AttnParams p = attention_params(B, Sq, Sk, E, H, scale);
    p.context = context;
    p.d_context = d_context;
    p.d_bias_q = d_bias_q;
    p.delta_out = delta_out;
    p.skip_score_gradient_store = store_score_gradient ? 0 : 1;

    CUtensorMap map_do, map_v, map_k, map_ds, map_dq, map_w;
    bool ok = make_map(&map_do, d_context, E, Sq, E, 1, 0, (int)B, Sq * E, 32, kQRows, false);
    ok = ok && make_map(&map_v, v, E, Sk, E, 1, 0, (int)B, Sk * E, 32, kMaxKeys, false);
    ok = ok && make_wide_map(&map_k, k, E, Sk, E, 1, 0, (int)B, Sk * E, HD / 32, kMaxKeys);
    ok = ok && make_map(&map_ds, d_scores, Sk, Sq, Sk, (int)H, Sq * Sk, (int)B, H * Sq * Sk, 32, 32, false, false);
    ok = ok && make_map(&map_dq, d_q, E, Sq, E, 1, 0, (int)B, Sq * E, 32, 32, false, false);
    ok = ok && make_map(&map_w, weights, Sk, Sq, Sk, (int)H, Sq * Sk, (int)B, H * Sq * Sk, 32, 32, false, false);
    if(!ok) return ONN_ERR_UNSUPPORTED;
    return launch_attention_core<true>(map_do, map_v, map_k, map_ds, map_dq, map_w, p, stream);
}

const unsigned int* attention_tc_status_word() { return tc::status_word_address(); }

int attention_tc_read_status()
{
    unsigned int status = 0;
    if(tc::read_and_clear_status(&status) != 0) return ONN_ERR_CUDA;
    return status == 0 ? ONN_OK : ONN_ERR_DEVICE_TIMEOUT;
}

}  // namespace onn
