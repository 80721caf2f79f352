// tcgen05 / TMA / mbarrier building blocks shared by the tensor-core kernels of this library: PTX wrappers,
// the shared-memory matrix descriptor, the time-limited barrier wait and the host code that encodes tensor maps.
//
// Every wait on an mbarrier is bounded: a wait that runs out records its site in this translation unit's
// device status word and raises the CTA's abort flag, which ends all role loops of the kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

namespace onn
{
namespace tc
{

constexpr unsigned long long kWaitCycles = 1ull << 31;     // ~1 s at 2 GHz

static __device__ unsigned int g_status;                   // per translation unit; 0 = ok, else the first failing wait site
// ---- PTX wrappers ----------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n" : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}

// Bounded wait.  Returns false (and raises the abort flag) if the barrier never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned int site,
                                          unsigned long long limit_cycles = kWaitCycles)
{
    if(mbar_try_wait(bar, parity)) return true;
    const unsigned long long start = clock64();
    unsigned int spins = 0;
    while(true)
    {
        if(mbar_try_wait(bar, parity)) return true;
        if((++spins & 255u) == 0)
        {
            if(*abort_flag) return false;
            if(clock64() - start > limit_cycles)
            {
                atomicCAS(&g_status, 0u, site);
                *abort_flag = 1;
                __threadfence_block();
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4)
{
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        :: "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 :: "l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 :: "l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}

__device__ __forceinline__ void tcgen05_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float* v)
{
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for(int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor, Blackwell version field = 1.
// layout_type: 2 = SWIZZLE_128B (K-major tiles), 1 = SWIZZLE_128B_BASE32B (MN-major tf32 tiles).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type)
{
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr >> 4) & 0x3FFF);          // start address, bits [0,14)
    desc |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;    // leading byte offset, bits [16,30)
    desc |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;    // stride byte offset, bits [32,46)
    desc |= (uint64_t)1 << 46;                              // descriptor version
    desc |= (uint64_t)layout_type << 61;
    return desc;
}

// ---- host side: tensor maps ---------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, []
    {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
           result == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

inline cuuint64_t stride_bytes(long long elements, long long fallback_elements)
{
    const long long e = elements > 0 ? elements : fallback_elements;
    return (cuuint64_t)e * 4ull;
}

// 4-D map (d0 = contiguous dimension, d1 = pitched dimension, batch inner, batch outer).
inline bool make_map(CUtensorMap* map, const float* base, long long d0, long long d1, long long pitch,
                     int batch_inner, long long stride_inner, int batch_outer, long long stride_outer,
                     int box0, int box1, bool mn_major, bool round_to_tf32 = true)
{
    EncodeTiledFn fn = encode_tiled();
    if(!fn) return false;
    const bool inner_on = batch_inner > 1 && stride_inner != 0, outer_on = batch_outer > 1 && stride_outer != 0;
    const cuuint64_t dims[4] = { (cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)(inner_on ? batch_inner : 1),
                                 (cuuint64_t)(outer_on ? batch_outer : 1) };
    const long long plane = pitch * d1;
    const cuuint64_t strides[3] = { (cuuint64_t)pitch * 4ull, stride_bytes(inner_on ? stride_inner : 0, plane),
                                    stride_bytes(outer_on ? stride_outer : 0, plane) };
    const cuuint32_t box[4] = { (cuuint32_t)box0, (cuuint32_t)box1, 1, 1 };
    const cuuint32_t elem[4] = { 1, 1, 1, 1 };
    return fn(map, round_to_tf32 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// MN-major operand whose contiguous extent is a multiple of 32: 5-D view (32 within an atom, reduction
// rows, atom index, batch inner, batch outer) so ONE copy brings [atoms][k_rows][32 floats],
// the same shared-memory image as `atoms` separate 4 KiB boxes.
inline bool make_wide_map(CUtensorMap* map, const float* base, long long mn, long long kdim, long long pitch,
                          int batch_inner, long long stride_inner, int batch_outer, long long stride_outer, int atoms, int k_rows)
{
    EncodeTiledFn fn = encode_tiled();
    if(!fn) return false;
    const bool inner_on = batch_inner > 1 && stride_inner != 0, outer_on = batch_outer > 1 && stride_outer != 0;
    const cuuint64_t dims[5] = { 32, (cuuint64_t)kdim, (cuuint64_t)(mn / 32), (cuuint64_t)(inner_on ? batch_inner : 1),
                                 (cuuint64_t)(outer_on ? batch_outer : 1) };
    const long long plane = pitch * kdim;
    const cuuint64_t strides[4] = { (cuuint64_t)pitch * 4ull, 128ull, stride_bytes(inner_on ? stride_inner : 0, plane),
                                    stride_bytes(outer_on ? stride_outer : 0, plane) };
    const cuuint32_t box[5] = { 32, (cuuint32_t)k_rows, (cuuint32_t)atoms, 1, 1 };
    const cuuint32_t elem[5] = { 1, 1, 1, 1, 1 };
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_TFLOAT32, 5, const_cast<float*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The status word belongs to the translation unit that includes this header (internal linkage), so the host functions
// that name it have internal linkage too: an `inline` function with external linkage would be merged across translation
// units by the linker and then read one unit's word for all of them.

// Reads and clears this translation unit's device status word (synchronises the device).
static inline int read_and_clear_status(unsigned int* status)
{
    unsigned int zero = 0;
    *status = 0;
    if(cudaDeviceSynchronize() != cudaSuccess) return -1;
    if(cudaMemcpyFromSymbol(status, g_status, sizeof(*status)) != cudaSuccess) return -1;
    if(*status != 0) cudaMemcpyToSymbol(g_status, &zero, sizeof(zero));
    return 0;
}

// Device address of this translation unit's status word on the current device (nullptr on failure), for kernels
// that look at it in stream order.
static inline const unsigned int* status_word_address()
{
    unsigned int* address = nullptr;
    if(cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_status) != cudaSuccess) return nullptr;
    return address;
}

}  // namespace tc
}  // namespace onn
