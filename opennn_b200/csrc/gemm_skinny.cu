// fp32 GEMM for a handful of rows: C[M,N] = alpha * A[M,K] W[K,N] (+ bias)(ReLU), M <= 64.
//
// One decoding step of the transformer multiplies [batch, 1, E] activations by every weight matrix of the decoder: the
// product is a weight stream, bound by HBM, and a 128-row tensor-core tile would give it to N/256 CTAs.  Here the weight
// matrix is cut into strips of 32 columns and each strip into 8 ranges of K; the 8 CTAs of a strip form a thread-block
// cluster, each streams its [K/8, 32] slab through a cp.async ring (the M rows of A with it), keeps a [MB, 32] partial
// tile in registers, and the cluster adds the 8 partial tiles through distributed shared memory in a fixed order --
// no workspace, no atomics, the same bits on every run.  A 1024 x 1024 matrix is read by 256 CTAs.
#include <cooperative_groups.h>

#include <cstdlib>

#include "common.cuh"
#include "gemm_internal.h"
#include "launch_counter.h"

namespace cg = cooperative_groups;

namespace onn
{
namespace skinny
{
constexpr int BN = 32, BK = 32, THREADS = 128, STAGES = 3, SPLITS = 8;
constexpr int A_PITCH = BK + 4;              // floats; keeps 16-byte alignment of every row

struct Params
{
    const float* A; const float* W; const float* bias; float* C;
    long long M, N, K, lda, ldb, ldc;
    long long k_chunk;                       // K range of one CTA, a multiple of BK
    float alpha;
    int relu, accumulate;
};

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid)
{
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;        // 0: the 16 bytes are filled with zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// RM rows per thread: the CTA holds MB = 16 * RM rows of A
template <int RM>
__global__ void __cluster_dims__(1, SPLITS, 1) __launch_bounds__(THREADS)
gemm_skinny_kernel(const Params p)
{
    constexpr int MB = 16 * RM;
    struct Stage { float w[BK][BN]; float a[MB][A_PITCH]; };
    __shared__ __align__(16) Stage stages[STAGES];
    static_assert(sizeof(Stage) * STAGES >= sizeof(float) * MB * BN, "the partial tile reuses the ring");
    static_assert(sizeof(Stage) * STAGES <= 48 * 1024, "static shared memory");

    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int tid = threadIdx.x, tx = tid & 7, ty = tid >> 3;
    const long long n0 = (long long)blockIdx.x * BN;
    const long long k_begin = rank * p.k_chunk;
    const long long k_end = p.K < k_begin + p.k_chunk ? p.K : k_begin + p.k_chunk;
    const int steps = k_end > k_begin ? (int)((k_end - k_begin + BK - 1) / BK) : 0;

    pdl_wait();

    auto load_stage = [&](int step)
    {
        Stage& s = stages[step % STAGES];
        const long long k0 = k_begin + (long long)step * BK;
#pragma unroll
        for(int i = 0; i < 2; i++)                       // W: BK rows of 8 float4
        {
            const int e = tid + i * THREADS, row = e >> 3, c4 = e & 7;
            const long long gk = k0 + row, gn = n0 + c4 * 4;
            const bool valid = gk < k_end && gn < p.N;
            cp_async_16(&s.w[row][c4 * 4], valid ? p.W + gk * p.ldb + gn : p.W, valid);
        }
#pragma unroll
        for(int i = 0; i < RM; i++)                      // A: MB rows of 8 float4
        {
            const int e = tid + i * THREADS, m = e >> 3, k4 = e & 7;
            const long long gk = k0 + k4 * 4;
            const bool valid = m < p.M && gk < k_end;
            cp_async_16(&s.a[m][k4 * 4], valid ? p.A + m * p.lda + gk : p.A, valid);
        }
    };

    float acc[RM][4] = {};

    for(int s = 0; s < STAGES - 1; s++)
    {
        if(s < steps) load_stage(s);
        cp_async_commit();
    }
    for(int step = 0; step < steps; step++)
    {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                                 // stage `step` has landed; everyone is done with stage step - 1
        if(step + STAGES - 1 < steps) load_stage(step + STAGES - 1);
        cp_async_commit();
        const Stage& s = stages[step % STAGES];
#pragma unroll
        for(int kk = 0; kk < BK; kk += 4)
        {
            float4 a[RM];
#pragma unroll
            for(int i = 0; i < RM; i++) a[i] = *reinterpret_cast<const float4*>(&s.a[ty * RM + i][kk]);
#pragma unroll
            for(int j = 0; j < 4; j++)
            {
                const float4 w = *reinterpret_cast<const float4*>(&s.w[kk + j][tx * 4]);
#pragma unroll
                for(int i = 0; i < RM; i++)
                {
                    const float av = j == 0 ? a[i].x : (j == 1 ? a[i].y : (j == 2 ? a[i].z : a[i].w));
                    acc[i][0] = fmaf(av, w.x, acc[i][0]);
                    acc[i][1] = fmaf(av, w.y, acc[i][1]);
                    acc[i][2] = fmaf(av, w.z, acc[i][2]);
                    acc[i][3] = fmaf(av, w.w, acc[i][3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                     // the ring is free: it now holds this CTA's partial tile
    pdl_launch_dependents();

    float (*partial)[BN] = reinterpret_cast<float (*)[BN]>(&stages[0]);
#pragma unroll
    for(int i = 0; i < RM; i++)
        *reinterpret_cast<float4*>(&partial[ty * RM + i][tx * 4]) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    cluster.sync();

    // CTA `rank` adds rows [rank * MB/8, (rank + 1) * MB/8) of the 8 partial tiles, always in the order 0..7
    constexpr int ROWS = MB / SPLITS;
    for(int o = tid; o < ROWS * BN; o += THREADS)
    {
        const int row = rank * ROWS + o / BN, col = o % BN;
        float sum = 0.f;
#pragma unroll
        for(int q = 0; q < SPLITS; q++)
        {
            const float (*remote)[BN] = reinterpret_cast<const float (*)[BN]>(cluster.map_shared_rank(&stages[0], q));
            sum += remote[row][col];
        }
        const long long n = n0 + col;
        if(row < p.M && n < p.N)
        {
            float value = p.alpha * sum;
            if(p.bias) value += p.bias[n];
            if(p.relu) value = fmaxf(value, 0.f);
            float* dst = p.C + row * p.ldc + n;
            *dst = p.accumulate ? *dst + value : value;
        }
    }
    cluster.sync();                                      // nobody leaves while its tile is still being read
}
}  // namespace skinny

bool gemm_skinny_takes(const onn_gemm_args& g)
{
    static const bool enabled = []{ const char* e = std::getenv("ONN_B200_GEMM_SKINNY"); return !(e && e[0] == '0'); }();
    if(!enabled || g.M > 64 || g.a_major != 0 || g.b_major != 1) return false;
    if(g.batch_inner != 1 || g.batch_outer != 1 || g.k_parts > 1 || g.split_k > 1) return false;
    if(g.relu_mask || g.relu_bits || g.relu_bits_out || g.colsum_out) return false;
    if((g.K & 3) || (g.N & 3) || (g.lda & 3) || (g.ldb & 3)) return false;
    if(((uintptr_t)g.A & 15) || ((uintptr_t)g.B & 15)) return false;
    // CUDA-core arithmetic: past ~1 GFLOP the tensor-core kernel wins even with most of its tile rows empty
    return g.M <= 16 || g.N * g.K <= (8LL << 20);
}

int gemm_skinny_launch(const onn_gemm_args& g, cudaStream_t stream)
{
    using namespace skinny;
    Params p;
    p.A = g.A; p.W = g.B; p.bias = g.bias; p.C = g.C;
    p.M = g.M; p.N = g.N; p.K = g.K; p.lda = g.lda; p.ldb = g.ldb; p.ldc = g.ldc;
    p.k_chunk = ((g.K + SPLITS - 1) / SPLITS + BK - 1) / BK * BK;
    p.alpha = g.alpha; p.relu = g.relu ? 1 : 0; p.accumulate = (g.flags & ONN_ACCUMULATE) ? 1 : 0;
    const dim3 grid((unsigned)((g.N + BN - 1) / BN), SPLITS, 1);
    cudaError_t status;
    if(g.M <= 16) status = launch_overlapped(gemm_skinny_kernel<1>, grid, dim3(THREADS), 0, stream, p);
    else if(g.M <= 32) status = launch_overlapped(gemm_skinny_kernel<2>, grid, dim3(THREADS), 0, stream, p);
    else status = launch_overlapped(gemm_skinny_kernel<4>, grid, dim3(THREADS), 0, stream, p);
    if(status != cudaSuccess) return ONN_ERR_CUDA;
    count_launch();
    return ONN_OK;
}

}  // namespace onn
