// Shared helpers for the sm_100a kernels: status codes, launch checks, warp/block
// reductions and 128-bit access helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdlib>
#include <mutex>
#include <utility>

#include "../../include/onn_b200.h"

namespace onn
{

constexpr int kSmCount = 148;   // B200: 2 dies x 74 SMs; grids are sized in multiples of this

// How many SMs the persistent kernels (one CTA or CTA pair per SM, most of the SM's shared memory each) may occupy;
// kSmCount unless a caller has asked for fewer with onn_set_sm_limit, e.g. to leave SMs to NCCL's kernels while a
// gradient bucket is being reduced.  Read on the host at launch time, so it takes effect in stream order.
int sm_limit();

// Work-item counters of the persistent kernels that can hand out their work items in the order the CTAs ask for them: a
// CTA that gets its SM late -- another kernel, e.g. one of NCCL's, holds it -- then takes fewer items instead of making
// the whole launch wait for a fixed share.  next_work_counter() returns the device address, on the current device, of a
// counter at zero, taken round robin from a pool; the kernel that uses it leaves it at zero (work_ring.cuh) and touches
// it only after it has waited for the launch before it on its stream, so two launches of one stream can share a counter
// (a graph replays the counters it was captured with, and the pool comes round to them).  Launches of DIFFERENT streams
// that run at the same time must not: with 8192 counters that takes a graph replay on one stream meeting, on another,
// the one eager launch in 8192 that drew the same counter -- callers that run this library on several streams at once
// keep the mode off.  Null -- fixed shares -- unless the mode is on
// (onn_set_dynamic_work; the data-parallel trainer turns it on).  reset_work_counters(): after a kernel gave up on a
// wait and left its counter behind.
unsigned int* next_work_counter();
void reset_work_counters();

#define ONN_CHECK_ARG(cond) do { if(!(cond)) return ONN_ERR_INVALID_ARGUMENT; } while(0)

inline int launch_status()
{
    return cudaGetLastError() == cudaSuccess ? ONN_OK : ONN_ERR_CUDA;
}

// A function attribute (the dynamic shared memory a kernel may use) belongs to the CURRENT device's copy of the
// function, so it is set once per device, before the first launch there that needs it.  One PerDeviceBytes per kernel.
constexpr int kMaxDevices = 64;
struct PerDeviceBytes { std::mutex lock; size_t bytes[kMaxDevices]; };

template <typename Kernel>
inline bool ensure_dynamic_smem(Kernel kernel, PerDeviceBytes& state, size_t wanted)
{
    int device = 0;
    if(cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return false;
    std::lock_guard<std::mutex> guard(state.lock);
    if(wanted <= state.bytes[device]) return true;
    if(wanted > 48 * 1024 &&
       cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)wanted) != cudaSuccess) return false;
    state.bytes[device] = wanted;
    return true;
}

inline int grid_for(long long work_items, int items_per_block, int blocks_per_sm)
{
    long long blocks = (work_items + items_per_block - 1) / items_per_block;
    const long long cap = (long long)kSmCount * blocks_per_sm;
    if(blocks > cap) blocks = cap;
    if(blocks < 1) blocks = 1;
    return (int)blocks;
}

// Programmatic dependent launch.  A kernel launched with launch_overlapped() may become resident while the kernel in
// front of it on the stream is still finishing: its CTAs take the SMs that kernel's CTAs have left, run their set-up
// (barrier initialisation, tensor-memory allocation) and then block in pdl_wait() until the whole preceding grid has
// completed and its memory is visible.  So every kernel launched that way calls pdl_wait() in ALL its threads before
// it reads or writes global memory, and pdl_launch_dependents() to let its own successor do the same.  Kernels launched
// the ordinary way keep the ordinary full serialisation on both sides.  ONN_B200_PDL=0 turns the attribute off.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled()
{
    static const bool enabled = []{ const char* e = std::getenv("ONN_B200_PDL"); return !(e && e[0] == '0'); }();
    return enabled;
}

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args)
{
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
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
