// Key and value gradients of the attention core in one kernel, by recomputation (head size 64):
//     dV = P^T dO,   dK = scale * dS^T Q,   dS = P * (dP - delta),   dP = dO V^T,   delta = rowsum(dO * O)
// Replaces, in back-propagation, the two batched GEMMs that read the [B, H, Sq, Sk] matrices P and dS again
// (opennn/multihead_attention_layer.cpp:843-887 computes them with cublasSgemmStridedBatched over materialised P and dS),
// and with them the need to write dS to HBM at all.
//
// Both products contract over the QUERIES, so the tiles are built key-major: a CTA owns 128 keys of one (batch, head) --
// the accumulator lanes -- and walks the queries in steps of 64 columns:
//     S^T  = K Q^T          (tcgen05.mma, tf32, [128 keys x 64 queries] in tensor memory)
//     dP^T = V dO^T         (same shape, beside it)
//     P^T  = exp2(S^T * scale * log2e [masks] - max_q) / sum_q      with the row maximum and sum of every query saved
//                                                                   by the forward kernel, so no [Sq, Sk] matrix is read
//     dS^T = P^T * (dP^T - delta_q)
//     dV  += P^T dO,  dK += dS^T Q   (second pair of MMAs: A operand straight from tensor memory, B = dO / Q MN-major)
// P^T and dS^T never leave the SM.  HBM traffic per (batch, head): K, V once; Q and dO once per key tile (from L2 after
// the first); dK and dV out once -- about 0.4 GB per layer of the benchmark network instead of 1.2 GB.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer (owns tensor memory), warps 2..9 = softmax arithmetic and output:
// two groups of four warps (one per accumulator quadrant) that take alternate steps, so that one computes while the other
// waits for tensor memory.  Two score buffers in tensor memory and two sets of query-side operands in shared memory: the
// score MMAs of step n + 1 run while step n is being worked on.  Every barrier wait is bounded (tcgen05.cuh).
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

constexpr int kKeyRows = 128;                            // keys per work item = accumulator lanes
constexpr int kStepQueries = 64;                         // queries per step = columns of one score buffer
constexpr int kGradHead = 64;

struct KvGradParams
{
    const unsigned char* key_is_pad;                      // [B, Sk] or null
    const float* row_max;                                 // [B, H, Sq] log2-domain row maximum the forward kernel saved
    const float* row_inv;                                 // [B, H, Sq] 1 / row sum
    const float* delta;                                   // [B, H, Sq] rowsum(dO * O), written by the query-gradient kernel
    float* d_k;                                           // [B, Sk, E]
    float* d_v;                                           // [B, Sk, E]
    float* d_bias_k;                                      // [E] column sums of dK are added here (may be null)
    float* d_bias_v;                                      // [E]
    int B, H, Sq, Sk, E;
    uint32_t key_tiles;                                   // ceil(Sk / 128)
    int query_steps;                                      // ceil(Sq / 64)
    int causal;
    float scale;
    uint32_t items;                                       // B * H * key_tiles
};

// Position in the sequence of steps every role walks: work items w = blockIdx.x, + gridDim.x, ...; within an item the
// query steps from the first that can see the key tile (causal: queries before the tile's first key see none of it).
// The divisions happen once per item, never per step.
struct Walk
{
    uint32_t w, item;                                     // work item and its running number in this CTA
    int qs, first;                                        // query step, and the item's first one
    int b, h, kt;
    bool valid;
};

__device__ __forceinline__ void enter_item(const KvGradParams& p, Walk& c)
{
    c.valid = c.w < p.items;
    if(!c.valid) return;
    // Items are ordered by key tile, the first tile of every head before the second ...: with a causal mask an item's
    // step count falls with its key tile, and this order gives every CTA the same mix of long and short items.
    const uint32_t heads = (uint32_t)p.B * (uint32_t)p.H;
    c.kt = (int)(c.w / heads);
    const uint32_t bh = c.w - (uint32_t)c.kt * heads;
    c.b = (int)(bh / (uint32_t)p.H);
    c.h = (int)(bh - (uint32_t)c.b * (uint32_t)p.H);
    c.first = p.causal ? c.kt * (kKeyRows / kStepQueries) : 0;
    c.qs = c.first;
}

__device__ __forceinline__ Walk first_walk(const KvGradParams& p)
{
    Walk c = {};
    c.w = blockIdx.x;
    enter_item(p, c);
    return c;
}

__device__ __forceinline__ void advance(const KvGradParams& p, Walk& c)
{
    if(++c.qs < p.query_steps) return;
    c.w += gridDim.x;
    c.item++;
    enter_item(p, c);
}

constexpr int kKvOperandBytes = 2 * kKeyRows * 128;                    // K or V tile, K-major: [2 k-blocks][128 rows][128 B]
constexpr int kQOperandBytes = 2 * kStepQueries * 128;                // one query-side operand of a step: 16 KiB
constexpr int kStageBytes = 4 * kQOperandBytes;                        // Q, dO K-major + Q, dO MN-major
constexpr int kKvGradSmem = 2 * kKvOperandBytes + 2 * kStageBytes + kSoftmaxWarps * 3 * kStepQueries * 4 + 1024 + 512;
static_assert(kKvGradSmem <= 232448, "beyond the shared memory of one CTA");

// lane L of the warp ends with the sum over the 32 lanes of v[L] (v is consumed)
__device__ __forceinline__ float column_sums_32(float* v, int lane)
{
#pragma unroll
    for(int width = 16; width >= 1; width >>= 1)
    {
        const bool upper = (lane & width) != 0;
#pragma unroll
        for(int i = 0; i < width; i++)
        {
            const float send = upper ? v[i] : v[i + width];
            const float keep = upper ? v[i + width] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, width);
        }
    }
    return v[0];
}

__global__ void __launch_bounds__(kAttnThreads, 1)
attention_kv_grad_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                         const __grid_constant__ CUtensorMap map_q_mn, const __grid_constant__ CUtensorMap map_do_mn, const KvGradParams p)
{
    constexpr int HD = kGradHead;
    constexpr uint32_t TMEM_COLS = 512;                  // score buffers 0..127 and 128..255 (S^T, dP^T of 64 columns each), dV 256.., dK 320..
    constexpr uint32_t DV_COL = 256, DK_COL = 320;
    // D = fp32, A = B = tf32, M = 128, N = 64: score MMAs (both operands K-major) and gradient MMAs (A from tensor memory, B MN-major)
    constexpr uint32_t IDESC_S = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kStepQueries >> 3) << 17) | ((uint32_t)(kKeyRows >> 4) << 24);
    constexpr uint32_t IDESC_G = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(kKeyRows >> 4) << 24);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* k_smem = smem;
    uint8_t* v_smem = k_smem + kKvOperandBytes;
    uint8_t* stage_smem = v_smem + kKvOperandBytes;      // [2 stages][Q K-major, dO K-major, Q MN-major, dO MN-major]
    float* column_stats = reinterpret_cast<float*>(stage_smem + 2 * kStageBytes);   // [8 warps][max, inv, delta][64 columns]
    uint64_t* bars = reinterpret_cast<uint64_t*>(column_stats + kSoftmaxWarps * 3 * kStepQueries);
    uint64_t* kv_full = bars + 0;
    uint64_t* kv_free = bars + 1;
    uint64_t* acc_full = bars + 2;
    uint64_t* acc_free = bars + 3;
    uint64_t* qk_full = bars + 4;                        // [2]
    uint64_t* qk_free = bars + 6;                        // [2]
    uint64_t* qm_full = bars + 8;                        // [2]
    uint64_t* qm_free = bars + 10;                       // [2]
    uint64_t* s_full = bars + 12;                        // [2]
    uint64_t* p_ready = bars + 14;                       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if(threadIdx.x == 0)
    {
        mbar_init(smem_u32(kv_full), 1); mbar_init(smem_u32(kv_free), 1);
        mbar_init(smem_u32(acc_full), 1); mbar_init(smem_u32(acc_free), kSoftmaxWarps);
        for(int s = 0; s < 2; s++)
        {
            mbar_init(smem_u32(qk_full + s), 1); mbar_init(smem_u32(qk_free + s), 1);
            mbar_init(smem_u32(qm_full + s), 1); mbar_init(smem_u32(qm_free + s), 1);
            mbar_init(smem_u32(s_full + s), 1); mbar_init(smem_u32(p_ready + s), kSoftmaxWarps / 2);
        }
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

    // All roles walk the same sequence of steps.  n counts steps over the whole kernel: stage and score buffer n & 1,
    // barrier parity (n >> 1) & 1.
    if(warp == 0)
    {
        // ---------------- TMA producer ----------------
        // Two independent streams of copies, polled in turn so that neither waits behind the other's barrier:
        //   `front`: K and V of an item, then per step the K-major Q / dO pair the score MMAs read
        //   `back` : per step the MN-major Q / dO pair the gradient MMAs read (freed a whole softmax round later)
        if(lane == 0)
        {
            Walk front = first_walk(p), back = front;
            uint32_t nf = 0, nb = 0;
            bool kv_loaded = false;
            int kv_armed = -1, qk_armed[2] = { -1, -1 }, qm_armed[2] = { -1, -1 };
            unsigned int idle = 0;
            unsigned long long idle_since = 0;
            while(front.valid || back.valid)
            {
                bool progress = false;
                if(front.valid)
                {
                    const uint32_t s = nf & 1u, parity = (nf >> 1) & 1u;
                    if(front.qs == front.first && !kv_loaded)
                    {
                        // K and V may be replaced once the previous item's last score MMAs have read them
                        if(mbar_try_wait(smem_u32(kv_free), (front.item & 1u) ^ 1u))
                        {
                            mbar_arrive_expect_tx(smem_u32(kv_full), 2 * kKvOperandBytes);
                            kv_armed = (int)(front.item & 1u);
#pragma unroll
                            for(int kb = 0; kb < 2; kb++)
                            {
                                tma_load_4d(smem_u32(k_smem + kb * kKeyRows * 128), &map_k, smem_u32(kv_full), front.h * HD + kb * 32, front.kt * kKeyRows, 0, front.b);
                                tma_load_4d(smem_u32(v_smem + kb * kKeyRows * 128), &map_v, smem_u32(kv_full), front.h * HD + kb * 32, front.kt * kKeyRows, 0, front.b);
                            }
                            kv_loaded = true;
                            progress = true;
                        }
                    }
                    else if(mbar_try_wait(smem_u32(qk_free + s), parity ^ 1u))   // the score MMAs of the step two back have run
                    {
                        uint8_t* stage = stage_smem + s * kStageBytes;
                        mbar_arrive_expect_tx(smem_u32(qk_full + s), 2 * kQOperandBytes);
                        qk_armed[s] = (int)parity;
#pragma unroll
                        for(int kb = 0; kb < 2; kb++)
                        {
                            tma_load_4d(smem_u32(stage + kb * kStepQueries * 128), &map_q, smem_u32(qk_full + s), front.h * HD + kb * 32, front.qs * kStepQueries, 0, front.b);
                            tma_load_4d(smem_u32(stage + kQOperandBytes + kb * kStepQueries * 128), &map_do, smem_u32(qk_full + s), front.h * HD + kb * 32, front.qs * kStepQueries, 0, front.b);
                        }
                        nf++;
                        advance(p, front);
                        kv_loaded = false;                   // only looked at on an item's first step
                        progress = true;
                    }
                }
                if(back.valid)
                {
                    const uint32_t s = nb & 1u, parity = (nb >> 1) & 1u;
                    if(mbar_try_wait(smem_u32(qm_free + s), parity ^ 1u))        // the gradient MMAs of the step two back have run
                    {
                        uint8_t* stage = stage_smem + s * kStageBytes;
                        mbar_arrive_expect_tx(smem_u32(qm_full + s), 2 * kQOperandBytes);
                        qm_armed[s] = (int)parity;
                        tma_load_5d(smem_u32(stage + 2 * kQOperandBytes), &map_q_mn, smem_u32(qm_full + s), 0, back.qs * kStepQueries, back.h * (HD / 32), 0, back.b);
                        tma_load_5d(smem_u32(stage + 3 * kQOperandBytes), &map_do_mn, smem_u32(qm_full + s), 0, back.qs * kStepQueries, back.h * (HD / 32), 0, back.b);
                        nb++;
                        advance(p, back);
                        progress = true;
                    }
                }
                if(progress) { idle = 0; continue; }
                // nothing was free: bounded like every other wait of the kernel
                if(idle == 0) idle_since = clock64();
                if((++idle & 255u) == 0)
                {
                    if(*abort_flag) break;
                    if(clock64() - idle_since > kWaitCycles)
                    {
                        atomicCAS(&g_status, 0u, 61u);
                        *abort_flag = 1;
                        __threadfence_block();
                        break;
                    }
                }
            }
            if(*abort_flag)
            {
                // no copy may still be writing this CTA's shared memory when it exits
                const auto drain = [](uint64_t* bar, int parity)
                {
                    if(parity < 0) return;
                    const unsigned long long start = clock64();
                    while(!mbar_try_wait(smem_u32(bar), (uint32_t)parity))
                        if(clock64() - start > kWaitCycles) break;
                };
                drain(kv_full, kv_armed);
                for(int s = 0; s < 2; s++) { drain(qk_full + s, qk_armed[s]); drain(qm_full + s, qm_armed[s]); }
            }
        }
    }
    else if(warp == 1)
    {
        // ---------------- MMA issuer ----------------
        if(lane == 0)
        {
            // descriptors of stage 0, k-block 0; every other one differs by a constant (addresses are in units of 16 bytes)
            const uint64_t k_desc = make_smem_desc(smem_u32(k_smem), 16, 1024, 2);
            const uint64_t v_desc = make_smem_desc(smem_u32(v_smem), 16, 1024, 2);
            const uint64_t qk_desc = make_smem_desc(smem_u32(stage_smem), 16, 1024, 2);
            const uint64_t qm_desc = make_smem_desc(smem_u32(stage_smem + 2 * kQOperandBytes), kStepQueries * 128, 512, 1);
            constexpr uint64_t kStageStep = kStageBytes >> 4, kOperandStep = kQOperandBytes >> 4;
            constexpr uint64_t kKeyBlockStep = (kKeyRows * 128) >> 4, kQueryBlockStep = (kStepQueries * 128) >> 4;

            // Issue order: scores(0); then for every step n: scores(n + 1), gradients(n).  The tensor pipe runs in order, so
            // scores(n + 2) overwrite a score buffer only after gradients(n) have read it.
            // The item's K and V must have landed before its first step, and may be replaced after its last one.
            const auto scores = [&](const Walk& c, uint32_t n) -> bool
            {
                const uint32_t s = n & 1u, parity = (n >> 1) & 1u;
                if(c.qs == c.first && !mbar_wait(smem_u32(kv_full), c.item & 1u, abort_flag, 65)) return false;
                if(!mbar_wait(smem_u32(qk_full + s), parity, abort_flag, 64)) return false;
                tcgen05_fence_after();
                const uint32_t acc = tmem_base + s * 128u;
                const uint64_t q_desc = qk_desc + s * kStageStep, do_desc = q_desc + kOperandStep;
#pragma unroll
                for(int kb = 0; kb < 2; kb++)
#pragma unroll
                    for(int j = 0; j < 4; j++)
                    {
                        const uint32_t accumulate = (kb > 0 || j > 0) ? 1u : 0u;
                        tcgen05_mma_tf32(acc, k_desc + (kb * kKeyBlockStep + j * 2), q_desc + (kb * kQueryBlockStep + j * 2), IDESC_S, accumulate);
                        tcgen05_mma_tf32(acc + 64u, v_desc + (kb * kKeyBlockStep + j * 2), do_desc + (kb * kQueryBlockStep + j * 2), IDESC_S, accumulate);
                    }
                tcgen05_commit(smem_u32(qk_free + s));
                tcgen05_commit(smem_u32(s_full + s));
                if(c.qs == p.query_steps - 1) tcgen05_commit(smem_u32(kv_free));
                return true;
            };

            // `cur` is the step whose gradients come next, `nxt` the one after it
            Walk cur = first_walk(p);
            if(cur.valid)
            {
                Walk nxt = cur;
                uint32_t n = 0;
                bool ok = scores(cur, 0);
                advance(p, nxt);
                while(ok)
                {
                    if(nxt.valid && !scores(nxt, n + 1)) break;

                    // gradients of step n
                    const uint32_t s = n & 1u, parity = (n >> 1) & 1u;
                    const bool first_of_item = cur.qs == cur.first, last_of_item = cur.qs == p.query_steps - 1;
                    if(!mbar_wait(smem_u32(qm_full + s), parity, abort_flag, 67)) break;
                    if(!mbar_wait(smem_u32(p_ready + s), parity, abort_flag, 68)) break;
                    // the previous item's dK and dV have been read out of the accumulators
                    if(first_of_item && !mbar_wait(smem_u32(acc_free), (cur.item & 1u) ^ 1u, abort_flag, 69)) break;
                    tcgen05_fence_after();
                    {
                        const uint64_t q_desc = qm_desc + s * kStageStep, do_desc = q_desc + kOperandStep;
                        const uint32_t acc = tmem_base + s * 128u;
#pragma unroll
                        for(int kk = 0; kk < kStepQueries / 8; kk++)       // 8 queries per MMA
                        {
                            const uint32_t accumulate = (!first_of_item || kk > 0) ? 1u : 0u;
                            tcgen05_mma_tf32_a_tmem(tmem_base + DV_COL, acc + (uint32_t)(kk * 8), do_desc + (uint64_t)(kk * 1024 >> 4), IDESC_G, accumulate);
                            tcgen05_mma_tf32_a_tmem(tmem_base + DK_COL, acc + 64u + (uint32_t)(kk * 8), q_desc + (uint64_t)(kk * 1024 >> 4), IDESC_G, accumulate);
                        }
                    }
                    tcgen05_commit(smem_u32(qm_free + s));
                    if(last_of_item) tcgen05_commit(smem_u32(acc_full));

                    n++;
                    cur = nxt;
                    if(!cur.valid) break;
                    advance(p, nxt);
                }
            }
        }
    }
    else
    {
        // ---------------- softmax arithmetic and output (warps 2..9) ----------------
        // Two groups of four warps (one warp per accumulator quadrant each): group g takes the steps with n & 1 == g, i.e.
        // always score buffer g, all 64 query columns of the step in two chunks of 32.  While one group waits for tensor
        // memory or for its MMAs, the other computes.
        const int quadrant = warp & 3;                       // accumulator lanes (keys) 32 * quadrant .. + 31
        const int half = (warp - 2) >> 2;                    // the group; also the 32 output columns this warp stores
        const uint32_t lane_base = tmem_base + ((uint32_t)(quadrant * 32) << 16);
        float* stats = column_stats + (warp - 2) * 3 * kStepQueries;   // this warp's [max, inv, delta][64 columns]
        const float to_log2 = p.scale * kLog2e;
        uint32_t n = 0;
        bool ok = true;

        // the statistics of a step's 64 query columns: two columns per lane, fetched one step of this group ahead
        float ahead[6] = { 0.f, 0.f, 0.f, 0.f, 0.f, 0.f };
        Walk look = first_walk(p);                           // this group's next step but one
        if(half == 1 && look.valid) advance(p, look);
        const auto fetch_stats = [&]()
        {
            if(!look.valid) return;
            const long long base = ((long long)look.b * p.H + look.h) * p.Sq;
#pragma unroll
            for(int j = 0; j < 2; j++)
            {
                const int q = look.qs * kStepQueries + j * 32 + lane;
                const bool live = q < p.Sq;
                ahead[j] = live ? __ldg(p.row_max + base + q) : 0.f;
                ahead[2 + j] = live ? __ldg(p.row_inv + base + q) : 0.f;      // 0: a query past the end gives P = 0
                ahead[4 + j] = live ? __ldg(p.delta + base + q) : 0.f;
            }
            advance(p, look);
            if(look.valid) advance(p, look);
        };
        fetch_stats();

        for(Walk it = first_walk(p); ok && it.valid; )
        {
            const int key0 = it.kt * kKeyRows + quadrant * 32;  // first key of this warp
            const int key = key0 + lane;
            const bool key_live = key < p.Sk;
            const bool key_padded = key_live && p.key_is_pad && p.key_is_pad[(long long)it.b * p.Sk + key] != 0;
            const float padded_score = -1e9f * kLog2e;

            for(int qs = it.first; qs < p.query_steps; qs++, n++)
            {
                if((n & 1u) != (uint32_t)half) continue;
                const uint32_t s = n & 1u, parity = (n >> 1) & 1u;
                __syncwarp();
#pragma unroll
                for(int j = 0; j < 2; j++)
                {
                    stats[j * 32 + lane] = ahead[j];
                    stats[kStepQueries + j * 32 + lane] = ahead[2 + j];
                    stats[2 * kStepQueries + j * 32 + lane] = ahead[4 + j];
                }
                __syncwarp();
                fetch_stats();                               // this group's next step: on its way while this one is worked on

                if(lane == 0) ok = mbar_wait(smem_u32(s_full + s), parity, abort_flag, 70);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if(!ok) break;
                tcgen05_fence_after();

#pragma unroll
                for(int chunk = 0; chunk < 2; chunk++)
                {
                    const int q0 = qs * kStepQueries + chunk * 32;     // first query column of this chunk
                    const uint32_t score_cols = lane_base + s * 128u + (uint32_t)(chunk * 32);
                    float sc[32], dp[32];
                    tmem_load_32_issue(score_cols, sc);
                    tmem_load_32_issue(score_cols + 64u, dp);
                    tmem_load_wait();
                    tmem_load_pin_32(sc);
                    tmem_load_pin_32(dp);

                    const float4* max4 = reinterpret_cast<const float4*>(stats + chunk * 32);
                    const float4* inv4 = reinterpret_cast<const float4*>(stats + kStepQueries + chunk * 32);
                    const float4* delta4 = reinterpret_cast<const float4*>(stats + 2 * kStepQueries + chunk * 32);
                    // a dead key row, or a block entirely above the causal diagonal: zeros; a block the diagonal crosses:
                    // per-element test; everything else takes the short path
                    const bool dead = !key_live || (p.causal && key0 > q0 + 31);
                    const bool diagonal = p.causal && key0 + 31 > q0;
                    if(dead)
                    {
#pragma unroll
                        for(int i = 0; i < 32; i++) { sc[i] = 0.f; dp[i] = 0.f; }
                    }
                    else
                    {
#pragma unroll
                        for(int i4 = 0; i4 < 8; i4++)
                        {
                            const float4 mx = max4[i4], iv = inv4[i4], dl = delta4[i4];
                            const float mxs[4] = { mx.x, mx.y, mx.z, mx.w }, ivs[4] = { iv.x, iv.y, iv.z, iv.w }, dls[4] = { dl.x, dl.y, dl.z, dl.w };
#pragma unroll
                            for(int k = 0; k < 4; k++)
                            {
                                const int i = i4 * 4 + k;
                                const float t = key_padded ? padded_score - mxs[k] : fmaf(sc[i], to_log2, -mxs[k]);
                                float pr = round_tf32(exp2_approx(t)) * ivs[k];
                                if(diagonal && key > q0 + i) pr = 0.f;
                                const float ds = pr * (dp[i] - dls[k]);
                                sc[i] = round_tf32(pr);
                                dp[i] = round_tf32(ds);
                            }
                        }
                    }
                    tmem_store_32_issue(score_cols, sc);
                    tmem_store_32_issue(score_cols + 64u, dp);
                }
                tmem_store_wait();
                tcgen05_fence_before();
                __syncwarp();
                if(lane == 0) mbar_arrive(smem_u32(p_ready + s));    // the gradient MMAs of this step may start
            }
            if(!ok) break;

            // dV and dK of this key tile: this warp's 32 x 32 blocks (columns 32 * half ..); every lane holds one key row
            if(lane == 0) ok = mbar_wait(smem_u32(acc_full), it.item & 1u, abort_flag, 71);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if(!ok) break;
            tcgen05_fence_after();
            float dv[32], dk[32];
            tmem_load_32_issue(lane_base + DV_COL + (uint32_t)(half * 32), dv);
            tmem_load_32_issue(lane_base + DK_COL + (uint32_t)(half * 32), dk);
            tmem_load_wait();
            tmem_load_pin_32(dv);
            tmem_load_pin_32(dk);
            tcgen05_fence_before();
            __syncwarp();
            if(lane == 0) mbar_arrive(smem_u32(acc_free));           // the accumulators may take the next item
            if(key0 < p.Sk)
            {
                const int column = it.h * HD + half * 32;
#pragma unroll
                for(int i = 0; i < 32; i++) dk[i] *= p.scale;
                if(key_live)
                {
                    // 128 contiguous bytes per lane and matrix
                    const long long at = ((long long)it.b * p.Sk + key) * p.E + column;
                    float4* out_v = reinterpret_cast<float4*>(p.d_v + at);
                    float4* out_k = reinterpret_cast<float4*>(p.d_k + at);
#pragma unroll
                    for(int q4 = 0; q4 < 8; q4++)
                    {
                        out_v[q4] = make_float4(dv[q4 * 4], dv[q4 * 4 + 1], dv[q4 * 4 + 2], dv[q4 * 4 + 3]);
                        out_k[q4] = make_float4(dk[q4 * 4], dk[q4 * 4 + 1], dk[q4 * 4 + 2], dk[q4 * 4 + 3]);
                    }
                }
                // rows past Sk hold zeros (their weights were written as zeros above), so the column sums may take all lanes
                if(p.d_bias_v) atomicAdd(p.d_bias_v + column + lane, column_sums_32(dv, lane));
                if(p.d_bias_k) atomicAdd(p.d_bias_k + column + lane, column_sums_32(dk, lane));
            }

            it.w += gridDim.x;
            it.item++;
            enter_item(p, it);
        }
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

bool attention_kv_grad_supported(const float* q, const float* k, const float* v, const float* d_context, const float* d_k, const float* d_v,
                                 long long B, long long Sq, long long Sk, long long E, long long H)
{
    if(H <= 0 || E % H != 0 || E / H != tc::kGradHead) return false;
    if(B >= 65536 || Sq >= (1LL << 24) || Sk >= (1LL << 24)) return false;
    if(B * H * ((Sk + tc::kKeyRows - 1) / tc::kKeyRows) >= (1LL << 31)) return false;
    if(!host_aligned16(q) || !host_aligned16(k) || !host_aligned16(v) || !host_aligned16(d_context) || !host_aligned16(d_k) || !host_aligned16(d_v)) return false;
    return tc::encode_tiled() != nullptr;
}

int attention_kv_grad_launch(const float* q, const float* k, const float* v, const float* d_context, const unsigned char* key_is_pad,
                             const float* row_max, const float* row_inv, const float* delta,
                             float* d_k, float* d_v, float* d_bias_k, float* d_bias_v,
                             long long B, long long Sq, long long Sk, long long E, long long H, int causal, float scale, cudaStream_t stream)
{
    using namespace tc;
    KvGradParams p = {};
    p.key_is_pad = key_is_pad; p.row_max = row_max; p.row_inv = row_inv; p.delta = delta;
    p.d_k = d_k; p.d_v = d_v; p.d_bias_k = d_bias_k; p.d_bias_v = d_bias_v;
    p.B = (int)B; p.H = (int)H; p.Sq = (int)Sq; p.Sk = (int)Sk; p.E = (int)E;
    // with a causal mask a key tile past the last query would have no step at all
    if(causal && Sk > Sq) return ONN_ERR_UNSUPPORTED;
    p.key_tiles = (uint32_t)((Sk + kKeyRows - 1) / kKeyRows);
    p.query_steps = (int)((Sq + kStepQueries - 1) / kStepQueries);
    p.causal = causal;
    p.scale = scale;
    p.items = (uint32_t)(B * H * (long long)p.key_tiles);

    CUtensorMap map_k, map_v, map_q, map_do, map_q_mn, map_do_mn;
    bool ok = make_map(&map_k, k, E, Sk, E, 1, 0, (int)B, Sk * E, 32, kKeyRows, false);
    ok = ok && make_map(&map_v, v, E, Sk, E, 1, 0, (int)B, Sk * E, 32, kKeyRows, false);
    ok = ok && make_map(&map_q, q, E, Sq, E, 1, 0, (int)B, Sq * E, 32, kStepQueries, false);
    ok = ok && make_map(&map_do, d_context, E, Sq, E, 1, 0, (int)B, Sq * E, 32, kStepQueries, false);
    ok = ok && make_wide_map(&map_q_mn, q, E, Sq, E, 1, 0, (int)B, Sq * E, kGradHead / 32, kStepQueries);
    ok = ok && make_wide_map(&map_do_mn, d_context, E, Sq, E, 1, 0, (int)B, Sq * E, kGradHead / 32, kStepQueries);
    if(!ok) return ONN_ERR_UNSUPPORTED;

    static PerDeviceBytes configured;
    if(!ensure_dynamic_smem(attention_kv_grad_kernel, configured, kKvGradSmem)) return ONN_ERR_CUDA;
    const int grid = (int)(p.items < (uint32_t)sm_limit() ? p.items : (uint32_t)sm_limit());
    const cudaError_t launched = launch_overlapped(attention_kv_grad_kernel, dim3(grid), dim3(kAttnThreads), kKvGradSmem, stream,
                                                   map_k, map_v, map_q, map_do, map_q_mn, map_do_mn, p);
    count_launch();
    return launched == cudaSuccess ? launch_status() : ONN_ERR_CUDA;
}

const unsigned int* attention_kv_grad_status_word() { return tc::status_word_address(); }

int attention_kv_grad_read_status()
{
    unsigned int status = 0;
    if(tc::read_and_clear_status(&status) != 0) return ONN_ERR_CUDA;
    return status == 0 ? ONN_OK : ONN_ERR_DEVICE_TIMEOUT;
}

}  // namespace onn
