// GEMM for a handful of rows: C[M,N] = alpha * A[M,K] W[K,N] (+ bias)(ReLU), M <= 64.  fp32 arithmetic up to 16 rows (and
// for a matrix narrower than 512 columns), tf32 mma with fp32 accumulation for 17 to 64 rows.
//
// One decoding step of the transformer multiplies [batch, 1, E] activations by every weight matrix of the decoder: the
// product is a weight stream, bound by HBM, and a 128-row tensor-core tile would give it to N/256 CTAs.  Here the weight
// matrix is cut into strips of 128 columns (64 for more than 16 rows, 32 for a narrow matrix) and, while the strips
// alone leave SMs idle, each strip into 2, 4 or 8 ranges of K; the CTAs of a strip form a thread-block cluster.  Each
// CTA streams its slab through a deep cp.async ring (the M rows of A with it); a thread keeps an 8 x 4 block of the
// tile in registers for its share of the K rows of every ring slot; the K shares inside the CTA, then the CTAs of the
// cluster (through distributed shared memory), are added in a fixed order -- no workspace, no atomics, the same bits
// on every run.  Measured on a B200 inside a CUDA graph (weights not in L2): 8 x 1024 x 1024 in 5.1 us, 8 x 1024 x 4096
// in 8.3 us, 8 x 4096 x 1024 in 10.5 us, against 1.5 us for an empty node; 64 rows take 7.8, 12 and 17.7 us with the mma
// variant below (11, 19 and 34 us on CUDA cores).  The tcgen05 kernel keeps vocabulary-sized matrices: its 1 KB TMA
// rows read DRAM three times faster.
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
constexpr int BK = 32, THREADS = 256;
constexpr int A_PITCH = BK + 4;              // floats; keeps 16-byte alignment of every row

constexpr int MAX_PROBLEMS = 4;      // products that share A, N, K and the epilogue options in one launch (grid z)

struct Params
{
    const float* A;
    const float* Ws[MAX_PROBLEMS]; const float* biases[MAX_PROBLEMS]; float* Cs[MAX_PROBLEMS]; long long ldcs[MAX_PROBLEMS];
    long long M, N, K, lda, ldb;
    long long k_chunk;                       // K range of one CTA, a multiple of BK
    float alpha;
    int relu, accumulate;
    int problems;                            // grid z
};

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid)
{
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;        // 0: the 16 bytes are filled with zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Cluster barrier with a relaxed arrive: it orders nothing (the default release would first wait for this thread's
// global stores of C to be performed), it only keeps every CTA resident until all have read each other's tiles.
__device__ __forceinline__ void cluster_exit_barrier()
{
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// One ring slot: BK rows of the strip and the same K range of the MB rows of A.
template <int MB, int BN> struct Stage { float w[BK][BN]; float a[MB][A_PITCH]; };
// ring depth: about 54 KB (narrow strips) or 110 KB (wide strips) of shared memory per CTA
template <int MB, int BN> __host__ __device__ constexpr int stages_for() { return (BN == 32 ? 54 : 110) * 1024 / (int)sizeof(Stage<MB, BN>); }

// The CTA computes an [MB, BN] tile over its K range.  A thread owns 8 rows x 4 columns of it (so a float4 of the strip
// read from shared memory feeds 32 FMAs); the 256 threads are BN/4 across, MB/8 down and KS = 8192/(MB*BN) deep: the
// BK rows of a ring slot are dealt to the KS slices, whose tiles are added in a fixed order at the end.
// SPLITS CTAs (a cluster along y) share a strip.
template <int MB, int BN, int SPLITS>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_kernel(const Params p)
{
    constexpr int STAGES = stages_for<MB, BN>(), TX = BN / 4, TY = MB / 8, KS = THREADS / (TX * TY), KPS = BK / KS;
    static_assert(TX * TY * KS == THREADS && KPS * KS == BK && KPS >= 1 && STAGES >= 3, "tile shape");
    using Stage = skinny::Stage<MB, BN>;
    extern __shared__ __align__(16) unsigned char ring[];
    Stage* stages = reinterpret_cast<Stage*>(ring);
    static_assert(sizeof(Stage) * STAGES >= sizeof(float) * (KS + 1) * MB * BN, "the partial tiles reuse the ring");

    const int rank = SPLITS > 1 ? (int)blockIdx.y : 0;      // the cluster spans the whole y extent of the grid
    const float* const W = p.Ws[blockIdx.z];
    const float* const bias = p.biases[blockIdx.z];
    float* const C = p.Cs[blockIdx.z];
    const long long ldc = p.ldcs[blockIdx.z];
    const int tid = threadIdx.x, tx = tid % TX, ty = (tid / TX) % TY, ks = tid / (TX * TY);
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
        for(int i = 0; i < BK * TX / THREADS; i++)       // W: BK rows of TX float4; a warp covers whole rows where it can
        {
            const int e = tid + i * THREADS, row = e / TX, c4 = e % TX;
            const long long gk = k0 + row, gn = n0 + c4 * 4;
            const bool valid = gk < k_end && gn < p.N;
            cp_async_16(&s.w[row][c4 * 4], valid ? W + gk * p.ldb + gn : W, valid);
        }
#pragma unroll
        for(int i = 0; i < (MB * 8 + THREADS - 1) / THREADS; i++)     // A: MB rows of 8 float4
        {
            const int e = tid + i * THREADS, m = e >> 3, k4 = e & 7;
            if(MB * 8 % THREADS != 0 && e >= MB * 8) break;
            const long long gk = k0 + k4 * 4;
            const bool valid = m < p.M && gk < k_end;
            cp_async_16(&s.a[m][k4 * 4], valid ? p.A + m * p.lda + gk : p.A, valid);
        }
    };

    float acc[8][4] = {};

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
        if constexpr(KPS % 4 == 0)
        {
            // four K rows at a time: the rows of A come as float4 (one shared-memory wavefront per row, broadcast)
#pragma unroll
            for(int j = 0; j < KPS; j += 4)
            {
                const int k = ks * KPS + j;
                float4 w[4];
#pragma unroll
                for(int q = 0; q < 4; q++) w[q] = *reinterpret_cast<const float4*>(&s.w[k + q][tx * 4]);
#pragma unroll
                for(int r = 0; r < 8; r++)
                {
                    const float4 a = *reinterpret_cast<const float4*>(&s.a[ty * 8 + r][k]);
                    acc[r][0] = fmaf(a.x, w[0].x, acc[r][0]); acc[r][1] = fmaf(a.x, w[0].y, acc[r][1]);
                    acc[r][2] = fmaf(a.x, w[0].z, acc[r][2]); acc[r][3] = fmaf(a.x, w[0].w, acc[r][3]);
                    acc[r][0] = fmaf(a.y, w[1].x, acc[r][0]); acc[r][1] = fmaf(a.y, w[1].y, acc[r][1]);
                    acc[r][2] = fmaf(a.y, w[1].z, acc[r][2]); acc[r][3] = fmaf(a.y, w[1].w, acc[r][3]);
                    acc[r][0] = fmaf(a.z, w[2].x, acc[r][0]); acc[r][1] = fmaf(a.z, w[2].y, acc[r][1]);
                    acc[r][2] = fmaf(a.z, w[2].z, acc[r][2]); acc[r][3] = fmaf(a.z, w[2].w, acc[r][3]);
                    acc[r][0] = fmaf(a.w, w[3].x, acc[r][0]); acc[r][1] = fmaf(a.w, w[3].y, acc[r][1]);
                    acc[r][2] = fmaf(a.w, w[3].z, acc[r][2]); acc[r][3] = fmaf(a.w, w[3].w, acc[r][3]);
                }
            }
        }
        else
        {
#pragma unroll
            for(int j = 0; j < KPS; j++)
            {
                const int k = ks * KPS + j;
                const float4 w = *reinterpret_cast<const float4*>(&s.w[k][tx * 4]);
#pragma unroll
                for(int r = 0; r < 8; r++)
                {
                    const float a = s.a[ty * 8 + r][k];
                    acc[r][0] = fmaf(a, w.x, acc[r][0]); acc[r][1] = fmaf(a, w.y, acc[r][1]);
                    acc[r][2] = fmaf(a, w.z, acc[r][2]); acc[r][3] = fmaf(a, w.w, acc[r][3]);
                }
            }
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();
    __syncthreads();                                     // the ring is free: it now holds the tiles of the KS slices

    float (*slices)[MB][BN] = reinterpret_cast<float (*)[MB][BN]>(ring);           // [KS] tiles, then the CTA's sum
    float (*partial)[BN] = reinterpret_cast<float (*)[BN]>(ring + sizeof(float) * KS * MB * BN);
#pragma unroll
    for(int r = 0; r < 8; r++)
        *reinterpret_cast<float4*>(&slices[ks][ty * 8 + r][tx * 4]) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    __syncthreads();

    auto finish = [&](int row, int col, float sum)
    {
        const long long n = n0 + col;
        if(row < p.M && n < p.N)
        {
            float value = p.alpha * sum;
            if(bias) value += bias[n];
            if(p.relu) value = fmaxf(value, 0.f);
            float* dst = C + row * ldc + n;
            *dst = p.accumulate ? *dst + value : value;
        }
    };

    // the CTA's tile: slices added in the order 0..KS-1
    for(int o = tid; o < MB * BN; o += THREADS)
    {
        const int row = o / BN, col = o % BN;
        float sum = 0.f;
#pragma unroll
        for(int q = 0; q < KS; q++) sum += slices[q][row][col];
        if constexpr(SPLITS == 1) finish(row, col, sum);
        else partial[row][col] = sum;
    }

    if constexpr(SPLITS > 1)
    {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        // CTA `rank` adds its 1/SPLITS of the tile's elements over the cluster, always in the order 0..SPLITS-1
        constexpr int SHARE = MB * BN / SPLITS;
        static_assert(SHARE * SPLITS == MB * BN, "the tile divides among the cluster");
        for(int o = tid; o < SHARE; o += THREADS)
        {
            const int element = rank * SHARE + o, row = element / BN, col = element % BN;
            float sum = 0.f;
#pragma unroll
            for(int q = 0; q < SPLITS; q++)
            {
                const float (*remote)[BN] = reinterpret_cast<const float (*)[BN]>(cluster.map_shared_rank(&partial[0][0], q));
                sum += remote[row][col];
            }
            finish(row, col, sum);
        }
        cluster_exit_barrier();                          // nobody leaves while its tile is still being read
    }
}

// ---------------------------------------------------------------------------------------------------------------
// 17 to 64 rows: the same weight stream, but the arithmetic (64 x K x N FMAs) no longer hides behind it on CUDA cores.
// This variant keeps the ring, the strips (64 columns) and the cluster reduction and does the products with
// mma.sync m16n8k8 on tf32 operands rounded to nearest from the fp32 values in shared memory (fp32 accumulation), as
// the tensor-core path of the large GEMMs does.  8 warps: MB/32 down (two 16-row tiles each), the rest across.
// ---------------------------------------------------------------------------------------------------------------
constexpr int MMA_BN = 64, MMA_W_PITCH = MMA_BN + 8;     // pitch 72: the four K rows a fragment load touches fall in distinct banks
template <int MB> struct MmaStage { float w[BK][MMA_W_PITCH]; float a[MB][A_PITCH]; };
template <int MB> __host__ __device__ constexpr int mma_stages() { return 110 * 1024 / (int)sizeof(MmaStage<MB>); }

__device__ __forceinline__ uint32_t to_tf32(float x)
{
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int MB, int SPLITS>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_mma_kernel(const Params p)
{
    constexpr int BN = MMA_BN, STAGES = mma_stages<MB>(), WM = MB / 32, WN = 8 / WM, NT = BN / (8 * WN);
    static_assert(WM >= 1 && WM * 32 == MB && NT >= 1 && STAGES >= 3, "tile shape");
    using Stage = MmaStage<MB>;
    extern __shared__ __align__(16) unsigned char ring[];
    Stage* stages = reinterpret_cast<Stage*>(ring);
    static_assert(sizeof(Stage) * STAGES >= sizeof(float) * MB * BN, "the partial tile reuses the ring");

    const int rank = SPLITS > 1 ? (int)blockIdx.y : 0;
    const float* const W = p.Ws[blockIdx.z];
    const float* const bias = p.biases[blockIdx.z];
    float* const C = p.Cs[blockIdx.z];
    const long long ldc = p.ldcs[blockIdx.z];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int warp_m = warp % WM, warp_n = warp / WM;
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
        for(int i = 0; i < BK * (BN / 4) / THREADS; i++)
        {
            const int e = tid + i * THREADS, row = e / (BN / 4), c4 = e % (BN / 4);
            const long long gk = k0 + row, gn = n0 + c4 * 4;
            const bool valid = gk < k_end && gn < p.N;
            cp_async_16(&s.w[row][c4 * 4], valid ? W + gk * p.ldb + gn : W, valid);
        }
#pragma unroll
        for(int i = 0; i < MB * 8 / THREADS; i++)
        {
            const int e = tid + i * THREADS, m = e >> 3, k4 = e & 7;
            const long long gk = k0 + k4 * 4;
            const bool valid = m < p.M && gk < k_end;
            cp_async_16(&s.a[m][k4 * 4], valid ? p.A + m * p.lda + gk : p.A, valid);
        }
    };

    float acc[2][NT][4] = {};

    for(int s = 0; s < STAGES - 1; s++)
    {
        if(s < steps) load_stage(s);
        cp_async_commit();
    }
    for(int step = 0; step < steps; step++)
    {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        if(step + STAGES - 1 < steps) load_stage(step + STAGES - 1);
        cp_async_commit();
        const Stage& s = stages[step % STAGES];
#pragma unroll
        for(int k8 = 0; k8 < BK; k8 += 8)
        {
            uint32_t a[2][4], b[NT][2];
#pragma unroll
            for(int mt = 0; mt < 2; mt++)
            {
                const int row = warp_m * 32 + mt * 16 + g;
                a[mt][0] = to_tf32(s.a[row][k8 + t]);
                a[mt][1] = to_tf32(s.a[row + 8][k8 + t]);
                a[mt][2] = to_tf32(s.a[row][k8 + t + 4]);
                a[mt][3] = to_tf32(s.a[row + 8][k8 + t + 4]);
            }
#pragma unroll
            for(int nt = 0; nt < NT; nt++)
            {
                const int col = (warp_n * NT + nt) * 8 + g;
                b[nt][0] = to_tf32(s.w[k8 + t][col]);
                b[nt][1] = to_tf32(s.w[k8 + t + 4][col]);
            }
#pragma unroll
            for(int mt = 0; mt < 2; mt++)
#pragma unroll
                for(int nt = 0; nt < NT; nt++) mma_tf32(acc[mt][nt], a[mt], b[nt]);
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();
    __syncthreads();                                     // the ring is free: it now holds this CTA's tile

    float (*partial)[BN] = reinterpret_cast<float (*)[BN]>(ring);
#pragma unroll
    for(int mt = 0; mt < 2; mt++)
#pragma unroll
        for(int nt = 0; nt < NT; nt++)
        {
            const int row = warp_m * 32 + mt * 16 + g, col = (warp_n * NT + nt) * 8 + 2 * t;
            *reinterpret_cast<float2*>(&partial[row][col]) = make_float2(acc[mt][nt][0], acc[mt][nt][1]);
            *reinterpret_cast<float2*>(&partial[row + 8][col]) = make_float2(acc[mt][nt][2], acc[mt][nt][3]);
        }

    auto finish = [&](int row, int col, float sum)
    {
        const long long n = n0 + col;
        if(row < p.M && n < p.N)
        {
            float value = p.alpha * sum;
            if(bias) value += bias[n];
            if(p.relu) value = fmaxf(value, 0.f);
            float* dst = C + row * ldc + n;
            *dst = p.accumulate ? *dst + value : value;
        }
    };

    if constexpr(SPLITS == 1)
    {
        __syncthreads();
        for(int o = tid; o < MB * BN; o += THREADS) finish(o / BN, o % BN, partial[o / BN][o % BN]);
    }
    else
    {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        constexpr int SHARE = MB * BN / SPLITS;
        for(int o = tid; o < SHARE; o += THREADS)
        {
            const int element = rank * SHARE + o, row = element / BN, col = element % BN;
            float sum = 0.f;
#pragma unroll
            for(int q = 0; q < SPLITS; q++)
            {
                const float (*remote)[BN] = reinterpret_cast<const float (*)[BN]>(cluster.map_shared_rank(&partial[0][0], q));
                sum += remote[row][col];
            }
            finish(row, col, sum);
        }
        cluster_exit_barrier();                          // nobody leaves while its tile is still being read
    }
}

// Launch with the cluster along y (and programmatic dependent launch, as every kernel of the step).
template <typename Kernel>
int launch_kernel(Kernel kernel, PerDeviceBytes& configured, size_t shared, int bn, int splits, const Params& p, cudaStream_t stream)
{
    if(!ensure_dynamic_smem(kernel, configured, shared)) return ONN_ERR_CUDA;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((unsigned)((p.N + bn - 1) / bn), splits, (unsigned)p.problems);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    attributes[1].id = cudaLaunchAttributeClusterDimension;
    attributes[1].val.clusterDim.x = 1;
    attributes[1].val.clusterDim.y = splits;
    attributes[1].val.clusterDim.z = 1;
    config.attrs = attributes;
    config.numAttrs = splits > 1 ? 2 : 1;
    if(cudaLaunchKernelEx(&config, kernel, p) != cudaSuccess) return ONN_ERR_CUDA;
    count_launch();
    return ONN_OK;
}

template <int MB, int SPLITS>
int launch_mma(const Params& p, cudaStream_t stream)
{
    static PerDeviceBytes configured;                    // per instantiation and device; the attribute belongs to the function
    return launch_kernel(gemm_skinny_mma_kernel<MB, SPLITS>, configured, sizeof(MmaStage<MB>) * mma_stages<MB>(), MMA_BN, SPLITS, p, stream);
}

template <int MB>
int launch_mma_splits(const Params& p, int splits, cudaStream_t stream)
{
    switch(splits)
    {
        case 1: return launch_mma<MB, 1>(p, stream);
        case 2: return launch_mma<MB, 2>(p, stream);
        case 4: return launch_mma<MB, 4>(p, stream);
        default: return launch_mma<MB, 8>(p, stream);
    }
}

template <int MB, int BN, int SPLITS>
int launch(const Params& p, cudaStream_t stream)
{
    static PerDeviceBytes configured;                    // per instantiation and device; the attribute belongs to the function
    return launch_kernel(gemm_skinny_kernel<MB, BN, SPLITS>, configured, sizeof(Stage<MB, BN>) * stages_for<MB, BN>(), BN, SPLITS, p, stream);
}

template <int MB, int BN>
int launch_splits(const Params& p, int splits, cudaStream_t stream)
{
    switch(splits)
    {
        case 1: return launch<MB, BN, 1>(p, stream);
        case 2: return launch<MB, BN, 2>(p, stream);
        case 4: return launch<MB, BN, 4>(p, stream);
        default: return launch<MB, BN, 8>(p, stream);
    }
}

inline int launch_shape(const Params& p, int bn, int splits, cudaStream_t stream)
{
    if(bn == 128) return p.M <= 8 ? launch_splits<8, 128>(p, splits, stream) : launch_splits<16, 128>(p, splits, stream);
    if(bn == 64) return p.M <= 32 ? launch_mma_splits<32>(p, splits, stream) : launch_mma_splits<64>(p, splits, stream);
    if(p.M <= 8) return launch_splits<8, 32>(p, splits, stream);
    if(p.M <= 16) return launch_splits<16, 32>(p, splits, stream);
    if(p.M <= 32) return launch_splits<32, 32>(p, splits, stream);
    return launch_splits<64, 32>(p, splits, stream);
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
    // 32-column strips read 128 bytes per matrix row: fine while the matrix is a few MB, well below the DRAM rate of
    // the tensor-core kernel's 1 KB TMA rows on a vocabulary-sized one (measured: 1.5 against 4.5 TB/s on 1024 x 32000)
    return g.N * g.K <= (8LL << 20);
}

int gemm_skinny_launch_shared_input(const onn_gemm_args* gs, int count, cudaStream_t stream)
{
    using namespace skinny;
    if(count < 1 || count > MAX_PROBLEMS) return ONN_ERR_INVALID_ARGUMENT;
    const onn_gemm_args& g = gs[0];
    // Strips of 128 columns (512 contiguous bytes of every matrix row per request) for up to 16 rows of A, of 64 columns
    // beyond (tf32 mma tiles), of 32 for a narrow matrix; K is split while the strips alone leave SMs idle and a CTA
    // keeps at least two steps, up to a cluster of 8 (16 measured no faster).
    const int bn = g.N < 512 ? 32 : (g.M > 16 ? 64 : 128);
    const long long strips = (g.N + bn - 1) / bn * count;
    const long long enough = bn == 128 ? 128 : 256;
    int splits = 1;
    while(splits < 8 && strips * splits < enough && g.K / (splits * 2) >= 2 * BK) splits *= 2;
    Params p = {};
    p.A = g.A;
    for(int i = 0; i < MAX_PROBLEMS; i++)
    {
        const onn_gemm_args& gi = gs[i < count ? i : 0];
        p.Ws[i] = gi.B; p.biases[i] = gi.bias; p.Cs[i] = gi.C; p.ldcs[i] = gi.ldc;
    }
    p.M = g.M; p.N = g.N; p.K = g.K; p.lda = g.lda; p.ldb = g.ldb;
    p.k_chunk = ((g.K + splits - 1) / splits + BK - 1) / BK * BK;
    p.alpha = g.alpha; p.relu = g.relu ? 1 : 0; p.accumulate = (g.flags & ONN_ACCUMULATE) ? 1 : 0;
    p.problems = count;
    return launch_shape(p, bn, splits, stream);
}

int gemm_skinny_launch(const onn_gemm_args& g, cudaStream_t stream) { return gemm_skinny_launch_shared_input(&g, 1, stream); }

}  // namespace onn
