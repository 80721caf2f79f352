// CUDA-core fp32 GEMM with the same contract as the tcgen05 kernel.  It serves operands
// that do not meet the TMA alignment rules (pitch or base not a multiple of 16 bytes, e.g.
// a Dense layer with 9 outputs) and is the on-device cross-check for the tensor-core path.
// 64x64 tile per CTA, 4x4 outputs per thread, K step 16, any strides, any batch.
#include "common.cuh"
#include "gemm_internal.h"
#include "launch_counter.h"

namespace onn
{

constexpr int kTile = 64, kStep = 16;

__global__ void __launch_bounds__(256)
gemm_simt_kernel(const onn_gemm_args g, int splits, long long k_per_split)
{
    __shared__ float As[kStep][kTile + 4];
    __shared__ float Bs[kStep][kTile + 4];

    const int z = blockIdx.z / splits, split = blockIdx.z % splits;
    const int zi = z % g.batch_inner, zo = z / g.batch_inner;
    const float* A = g.A + zi * g.a_stride_inner + zo * g.a_stride_outer;
    const float* B = g.B + zi * g.b_stride_inner + zo * g.b_stride_outer;
    const long long c_offset = zi * g.c_stride_inner + zo * g.c_stride_outer;
    float* C = g.C + c_offset;
    const float* mask = g.relu_mask ? g.relu_mask + c_offset : nullptr;

    const long long m0 = (long long)blockIdx.y * kTile, n0 = (long long)blockIdx.x * kTile;
    const long long k_begin = split * k_per_split;
    const long long k_end = (long long)g.K < k_begin + k_per_split ? (long long)g.K : k_begin + k_per_split;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

    float acc[4][4] = {};

    for(long long k0 = k_begin; k0 < k_end; k0 += kStep)
    {
        // each thread fetches 4 elements of A and 4 of B, walking the contiguous dimension fastest
#pragma unroll
        for(int i = 0; i < 4; i++)
        {
            const int e = threadIdx.x + i * 256;
            int m, k;
            if(g.a_major == 0) { k = e & (kStep - 1); m = e / kStep; } else { m = e & (kTile - 1); k = e / kTile; }
            const long long gm = m0 + m, gk = k0 + k;
            float value = 0.f;
            if(gm < g.M && gk < k_end) value = g.a_major == 0 ? A[gm * g.lda + gk] : A[gk * g.lda + gm];
            As[k][m] = value;

            int n;
            if(g.b_major == 0) { k = e & (kStep - 1); n = e / kStep; } else { n = e & (kTile - 1); k = e / kTile; }
            const long long gn = n0 + n, gk2 = k0 + k;
            value = 0.f;
            if(gn < g.N && gk2 < k_end) value = g.b_major == 0 ? B[gn * g.ldb + gk2] : B[gk2 * g.ldb + gn];
            Bs[k][n] = value;
        }
        __syncthreads();
#pragma unroll
        for(int k = 0; k < kStep; k++)
        {
            float a[4], b[4];
#pragma unroll
            for(int i = 0; i < 4; i++) { a[i] = As[k][ty * 4 + i]; b[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
            for(int i = 0; i < 4; i++)
#pragma unroll
                for(int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }

    const bool accumulate = (g.flags & ONN_ACCUMULATE) != 0;
#pragma unroll
    for(int i = 0; i < 4; i++)
    {
        const long long m = m0 + ty * 4 + i;
        if(m >= g.M) continue;
#pragma unroll
        for(int j = 0; j < 4; j++)
        {
            const long long n = n0 + tx * 4 + j;
            if(n >= g.N) continue;
            float value = g.alpha * acc[i][j];
            if(g.bias && split == 0) value += g.bias[n];
            if(g.relu) value = fmaxf(value, 0.f);
            if(mask && !(mask[m * g.ldc + n] > 0.f)) value = 0.f;
            if(g.relu_bits && !((g.relu_bits[m * g.relu_bits_ld + (n >> 5)] >> (n & 31)) & 1u)) value = 0.f;
            // the bit matrix was cleared by the launcher; each thread sets the bits of its positive values
            if(g.relu_bits_out && value > 0.f) atomicOr(g.relu_bits_out + m * g.relu_bits_ld + (n >> 5), 1u << (n & 31));
            float* dst = C + m * g.ldc + n;
            if(splits > 1) atomicAdd(dst, value);
            else *dst = accumulate ? *dst + value : value;
            if(g.colsum_out) atomicAdd(g.colsum_out + zi * g.colsum_stride_inner + n, value);
        }
    }
}

int gemm_simt_launch(const onn_gemm_args& g, cudaStream_t stream)
{
    const int splits = g.split_k > 1 ? g.split_k : 1;
    long long k_per_split = (g.K + splits - 1) / splits;
    k_per_split = (k_per_split + kStep - 1) / kStep * kStep;
    const long long batch = (long long)g.batch_inner * g.batch_outer;
    if(batch * splits > 65535) return ONN_ERR_UNSUPPORTED;
    dim3 grid((unsigned)((g.N + kTile - 1) / kTile), (unsigned)((g.M + kTile - 1) / kTile), (unsigned)(batch * splits));
    if(grid.y > 65535) return ONN_ERR_UNSUPPORTED;
    if(g.relu_bits_out &&
       cudaMemsetAsync(g.relu_bits_out, 0, (size_t)g.M * (size_t)g.relu_bits_ld * sizeof(uint32_t), stream) != cudaSuccess)
        return ONN_ERR_CUDA;
    gemm_simt_kernel<<<grid, 256, 0, stream>>>(g, splits, k_per_split);
    count_launch();
    return launch_status();
}

}  // namespace onn
