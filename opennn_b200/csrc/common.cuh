// Shared helpers for the sm_100a kernels: status codes, launch checks, warp/block
// reductions, 128-bit access helpers and the fp32 -> tf32 round-to-nearest used by every
// kernel that produces a tensor-core operand.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/onn_b200.h"

namespace onn
{

constexpr int kSmCount = 148;   // B200: 2 dies x 74 SMs; grids are sized in multiples of this

#define ONN_CHECK_ARG(cond) do { if(!(cond)) return ONN_ERR_INVALID_ARGUMENT; } while(0)

inline int launch_status()
{
    return cudaGetLastError() == cudaSuccess ? ONN_OK : ONN_ERR_CUDA;
}

inline int grid_for(long long work_items, int items_per_block, int blocks_per_sm)
{
    long long blocks = (work_items + items_per_block - 1) / items_per_block;
    const long long cap = (long long)kSmCount * blocks_per_sm;
    if(blocks > cap) blocks = cap;
    if(blocks < 1) blocks = 1;
    return (int)blocks;
}

// Round an fp32 value to the nearest tf32-representable value (10 explicit mantissa bits),
// ties away from zero, kept in an fp32 container.  tcgen05 kind::tf32 ignores the low 13
// mantissa bits of its operands (truncation, a biased error); producers therefore store
// operands already rounded so the tensor cores see an unbiased 2^-11 relative error.
__device__ __forceinline__ float round_tf32(float x)
{
    uint32_t bits;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x));
    return __uint_as_float(bits);
}

__device__ __forceinline__ float maybe_round(float x, bool round)
{
    return round ? round_tf32(x) : x;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for(int offset = 16; offset > 0; offset >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for(int offset = 16; offset > 0; offset >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Block-wide sum for blocks of up to 1024 threads; `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if(lane == 0) scratch[warp] = v;
    __syncthreads();
    const int warps = (blockDim.x + 31) >> 5;
    v = (threadIdx.x < warps) ? scratch[threadIdx.x] : 0.0f;
    if(warp == 0) v = warp_sum(v);
    if(threadIdx.x == 0) scratch[0] = v;
    __syncthreads();
    return scratch[0];
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

// Streaming variants: data that is read or written once should not displace reused lines.
__device__ __forceinline__ float4 ld4_stream(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void st4_stream(float* p, float4 v) { __stcs(reinterpret_cast<float4*>(p), v); }

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline bool host_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Token ids and targets are floats holding integers; the reference converts with
// static_cast<Index>(float), i.e. truncation toward zero.
__device__ __forceinline__ long long token_index(float id) { return (long long)id; }

}  // namespace onn
