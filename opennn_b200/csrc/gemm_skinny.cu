// fp32 GEMM for a handful of rows: C[M,N] = alpha * A[M,K] W[K,N] (+ bias)(ReLU), M <= 64.
//
// One decoding step of the transformer multiplies [batch, 1, E] activations by every weight matrix of the decoder: the
// product is a weight stream, bound by HBM, and a 128-row tensor-core tile would give it to N/256 CTAs.  Here the weight
// matrix is cut into strips of 32 columns and, while that gives fewer than two CTAs per SM, each strip into 2, 4 or 8
// ranges of K; the CTAs of a strip form a thread-block cluster, each streams its slab through a deep cp.async ring (the
// M rows of A with it), keeps a [MB, 32] partial tile in registers, and the cluster adds the partial tiles through
// distributed shared memory in a fixed order -- no workspace, no atomics, the same bits on every run.  A 1024 x 1024
// matrix is read by 256 CTAs, each with ~50 KB of loads in flight.
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
constexpr int BN = 32, BK = 32, THREADS = 128;
constexpr int A_PITCH = BK + 4;              // floats; keeps 16-byte alignment of every row
// ring depth by rows per thread: about 50 KB of shared memory per CTA in every variant
__host__ __device__ constexpr int stages_for(int rm) { return rm == 1 ? 8 : (rm == 2 ? 6 : 4); }

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

template <int RM> struct Stage { float w[BK][BN]; float a[16 * RM][A_PITCH]; };

// RM rows per thread: the CTA holds MB = 16 * RM rows of A.  SPLITS CTAs (a cluster along y) share a strip.
template <int RM, int SPLITS>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const Params p)
{
    constexpr int MB = 16 * RM, STAGES = stages_for(RM);
    using Stage = skinny::Stage<RM>;
    extern __shared__ __align__(16) unsigned char ring[];
    Stage* stages = reinterpret_cast<Stage*>(ring);
    static_assert(sizeof(Stage) * STAGES >= sizeof(float) * MB * BN, "the partial tile reuses the ring");

    const int rank = SPLITS > 1 ? (int)blockIdx.y : 0;      // the cluster spans the whole y extent of the grid
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
    pdl_launch_dependents();

    if constexpr(SPLITS == 1)
    {
#pragma unroll
        for(int i = 0; i < RM; i++)
        {
            const int row = ty * RM + i;
            if(row >= p.M) continue;
#pragma unroll
            for(int j = 0; j < 4; j++)
            {
                const long long n = n0 + tx * 4 + j;
                if(n >= p.N) continue;
                float value = p.alpha * acc[i][j];
                if(p.bias) value += p.bias[n];
                if(p.relu) value = fmaxf(value, 0.f);
                float* dst = p.C + row * p.ldc + n;
                *dst = p.accumulate ? *dst + value : value;
            }
        }
    }
    else
    {
    cg::cluster_group cluster = cg::this_cluster();
    __syncthreads();                                     // the ring is free: it now holds this CTA's partial tile
    float (*partial)[BN] = reinterpret_cast<float (*)[BN]>(&stages[0]);
#pragma unroll
    for(int i = 0; i < RM; i++)
        *reinterpret_cast<float4*>(&partial[ty * RM + i][tx * 4]) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    cluster.sync();

    // CTA `rank` adds rows [rank * MB/SPLITS, (rank + 1) * MB/SPLITS) of the partial tiles, always in the order 0..SPLITS-1
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

namespace skinny
{
template <int RM, int SPLITS>
int launch(const Params& p, cudaStream_t stream)
{
    constexpr size_t shared = sizeof(Stage<RM>) * stages_for(RM);
    static bool configured = false;                      // per instantiation; the attribute belongs to the function
    if(!configured)
    {
        if(cudaFuncSetAttribute(gemm_skinny_kernel<RM, SPLITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared) != cudaSuccess)
            return ONN_ERR_CUDA;
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)((p.N + BN - 1) / BN), SPLITS, 1);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    attributes[1].id = cudaLaunchAttributeClusterDimension;
    attributes[1].val.clusterDim.x = 1;
    attributes[1].val.clusterDim.y = SPLITS;
    attributes[1].val.clusterDim.z = 1;
    config.attrs = attributes;
    config.numAttrs = SPLITS > 1 ? 2 : 1;
    if(cudaLaunchKernelEx(&config, gemm_skinny_kernel<RM, SPLITS>, p) != cudaSuccess) return ONN_ERR_CUDA;
    count_launch();
    return ONN_OK;
}

template <int RM>
int launch_rows(const Params& p, int splits, cudaStream_t stream)
{
    switch(splits)
    {
        case 1: return launch<RM, 1>(p, stream);
        case 2: return launch<RM, 2>(p, stream);
        case 4: return launch<RM, 4>(p, stream);
        default: return launch<RM, 8>(p, stream);
    }
}
}  // namespace skinny

int gemm_skinny_launch(const onn_gemm_args& g, cudaStream_t stream)
{
    using namespace skinny;
    // split K while the strips alone give fewer than two CTAs per SM and a CTA keeps at least two steps
    const long long strips = (g.N + BN - 1) / BN;
    int splits = 1;
    while(splits < 8 && strips * splits < 296 && g.K / (splits * 2) >= 2 * BK) splits *= 2;
    Params p;
    p.A = g.A; p.W = g.B; p.bias = g.bias; p.C = g.C;
    p.M = g.M; p.N = g.N; p.K = g.K; p.lda = g.lda; p.ldb = g.ldb; p.ldc = g.ldc;
    p.k_chunk = ((g.K + splits - 1) / splits + BK - 1) / BK * BK;
    p.alpha = g.alpha; p.relu = g.relu ? 1 : 0; p.accumulate = (g.flags & ONN_ACCUMULATE) ? 1 : 0;
    if(g.M <= 16) return launch_rows<1>(p, splits, stream);
    if(g.M <= 32) return launch_rows<2>(p, splits, stream);
    return launch_rows<4>(p, splits, stream);
}

}  // namespace onn
