// Building blocks shared by the fused attention kernels (attention_tc.cu: source lengths up to 256, one accumulator
// row per query; attention_long.cu: longer sources, walked in key tiles of 256): shapes, parameters, tensor-memory
// loads and stores that can be kept in flight, the tf32 rounding and exponential used by the softmax warps, the
// work-item order and the staged 32 x 32 block store.
#pragma once
#include "common.cuh"
#include "tcgen05.cuh"

namespace onn
{
namespace tc
{

constexpr int kSoftmaxWarps = 8;
constexpr int kAttnThreads = 64 + 32 * kSoftmaxWarps;     // 320
constexpr int kQRows = 128;                               // query rows per tile = accumulator lanes
constexpr int kMaxKeys = 256;                             // accumulator columns of one score row
constexpr int kHalfKeys = kMaxKeys / 2;                   // columns one softmax thread owns
constexpr int kBlock = 32 * 32 * 4;                       // one warp's 32 x 32 staging block
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams
{
    const unsigned char* key_is_pad;                      // [B, Sk] or null
    int B, H, Sq, Sk;
    int q_tiles;                                          // ceil(Sq / 128)
    int key_blocks;                                       // ceil(Sk / 32)
    int key_tiles;                                        // ceil(Sk / 256): tiles the long-source kernels walk (else unused)
    int causal;
    float scale;
    long long items;                                      // B * H * q_tiles
    // backward only
    const float* context;                                 // [B, Sq, E] forward output of the core
    const float* d_context;                               // [B, Sq, E] its gradient
    float* d_bias_q;                                      // [E]: column sums of dQ are added here (may be null)
    long long E;
    // hand-over to the key / value gradient kernel (attention_kv_grad.cu), all [B, H, Sq]; null = not wanted
    float* row_max_out;                                   // forward: log2-domain maximum of every query row, masks applied
    float* row_inv_out;                                   // forward: 1 / sum of the row's tf32-rounded exponentials
    float* delta_out;                                     // backward: rowsum(dO * O)
    int skip_score_gradient_store;                        // backward: dS stays on the SM (nobody reads it from HBM)
    unsigned int* work_counter;                           // items in the order the CTAs ask for them (work_ring.cuh); null: a fixed share per CTA
};

#define ONN_LIST8(M, v, o) M(v[(o)]), M(v[(o) + 1]), M(v[(o) + 2]), M(v[(o) + 3]), M(v[(o) + 4]), M(v[(o) + 5]), M(v[(o) + 6]), M(v[(o) + 7])
#define ONN_LIST32(M, v) ONN_LIST8(M, v, 0), ONN_LIST8(M, v, 8), ONN_LIST8(M, v, 16), ONN_LIST8(M, v, 24)
#define ONN_OUT_F(x) "=f"(x)
#define ONN_INOUT_F(x) "+f"(x)
#define ONN_IN_F(x) "f"(x)

// Issues a 32-column tensor-memory load WITHOUT waiting for it: several can be in flight at once.
__device__ __forceinline__ void tmem_load_32_issue(uint32_t taddr, float* v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : ONN_LIST32(ONN_OUT_F, v) : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// After the wait: an empty volatile statement that "rewrites" the loaded registers, so that no instruction
// consuming them can be scheduled above the wait.
__device__ __forceinline__ void tmem_load_pin_32(float* v) { asm volatile("" : ONN_LIST32(ONN_INOUT_F, v) :: "memory"); }

__device__ __forceinline__ void tmem_store_32_issue(uint32_t taddr, const float* v)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :: "r"(taddr), ONN_LIST32(ONN_IN_F, v) : "memory");
}

__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_mma_tf32_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n"
        "}\n" :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// fp32 -> nearest tf32 (ties away from zero) for finite x, as the bits of an fp32 value: add half a tf32 ulp to the
// magnitude and drop the 13 low mantissa bits.  Two integer instructions at full rate; the conversion instruction
// would share the quarter-rate unit with the exponentials.
__device__ __forceinline__ float round_tf32(float x)
{
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

__device__ __forceinline__ float exp2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void pair_barrier(int quadrant)
{
    // the two warps that share accumulator quadrant `quadrant` (64 threads); barrier 0 is __syncthreads
    asm volatile("bar.sync %0, 64;" :: "r"(1 + quadrant) : "memory");
}

struct AttnItem { int b, h, q_tile; };

__device__ __forceinline__ AttnItem decode_item(const AttnParams& p, long long w)
{
    // the query tiles of one head are neighbours, so the second one finds K and V in L2
    AttnItem it;
    it.q_tile = (int)(w % p.q_tiles); w /= p.q_tiles;
    // With a causal mask over several key tiles a query tile's work grows with its index, and a CTA that strides through
    // the items by the grid size would keep meeting the same few tile indices (148 and 8 query tiles: only t and t + 4).
    // Rotating the tile order of each head by roughly the round in which the head is reached lets every CTA meet all of
    // them; within a head it is still a permutation.
    if(p.causal && p.key_tiles > 1) it.q_tile = (int)((it.q_tile + (w * p.q_tiles) / gridDim.x) % p.q_tiles);
    it.h = (int)(w % p.H);
    it.b = (int)(w / p.H);
    return it;
}

// hands one staged 32 x 32 block (this warp's rows) to the copy engine
__device__ __forceinline__ void stage_and_store(const CUtensorMap* map, uint32_t warp_blocks, unsigned int& staged, const float* v, float factor,
                                                int lane, int c0, int c1, int c2, int c3)
{
    const uint32_t block = warp_blocks + (staged & 1u) * kBlock;
    // a block is free again once the copy issued from it two blocks ago has finished READING shared memory
    if(staged >= 2) { if(lane == 0) bulk_wait_read_1(); __syncwarp(); }
#pragma unroll
    for(int q4 = 0; q4 < 8; q4++)
    {
        // row `lane` of the block is 128 bytes; 16-byte chunk q4 goes to slot q4 ^ (lane % 8): the 128-byte swizzle
        const uint32_t dst = block + (uint32_t)lane * 128u + (uint32_t)((q4 ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(dst), "f"(v[q4 * 4] * factor), "f"(v[q4 * 4 + 1] * factor),
                     "f"(v[q4 * 4 + 2] * factor), "f"(v[q4 * 4 + 3] * factor));
    }
    fence_async_shared();
    __syncwarp();
    if(lane == 0) { tma_store_4d(map, block, c0, c1, c2, c3); bulk_commit(); }
    staged++;
}

}  // namespace tc
}  // namespace onn
