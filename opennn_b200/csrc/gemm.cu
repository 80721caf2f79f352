// Front end of the GEMM primitive: argument checks, choice between the tcgen05 kernel and
// the CUDA-core kernel, library-wide bookkeeping (launch counter, status strings).
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "gemm_internal.h"
#include "attention_internal.h"
#include "launch_counter.h"
#include "rowwise_internal.h"

namespace onn
{

std::atomic<uint64_t> g_launch_count{0};

// 0 unless a test has asked for one kernel family (onn_gemm_set_mode): the tensor-core kernel runs wherever the operands
// meet the TMA alignment rules, the CUDA-core kernel takes the rest
static std::atomic<int> g_mode{0};
static std::atomic<int> g_sm_limit{kSmCount};

int sm_limit() { return g_sm_limit.load(std::memory_order_relaxed); }

constexpr int kWorkCounters = 8192;
static __device__ unsigned int g_work_counters[kWorkCounters];
// -1: as the environment says (ONN_B200_DYNAMIC_WORK=1), else off; 0 / 1: set by onn_set_dynamic_work
static std::atomic<int> g_dynamic_work{-1};

static unsigned int* work_counters_of_current_device()
{
    static std::mutex mutex;
    static unsigned int* resolved[kMaxDevices] = {};
    int device = -1;
    if(cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    if(!resolved[device])
    {
        unsigned int* found = nullptr;
        if(cudaGetSymbolAddress(reinterpret_cast<void**>(&found), g_work_counters) != cudaSuccess) return nullptr;
        resolved[device] = found;
    }
    return resolved[device];
}

unsigned int* next_work_counter()
{
    static const int from_environment = []{ const char* e = std::getenv("ONN_B200_DYNAMIC_WORK"); return e ? (e[0] == '1' ? 1 : 0) : -1; }();
    const int mode = g_dynamic_work.load(std::memory_order_relaxed);
    const bool enabled = from_environment >= 0 ? from_environment == 1 : mode == 1;
    if(!enabled) return nullptr;
    static std::atomic<unsigned long long> sequence{0};
    unsigned int* base = work_counters_of_current_device();
    return base ? base + (sequence++ % kWorkCounters) : nullptr;
}

void reset_work_counters()
{
    if(unsigned int* base = work_counters_of_current_device()) cudaMemset(base, 0, sizeof(unsigned int) * kWorkCounters);
}

int gemm_mode() { return g_mode.load(std::memory_order_relaxed); }

// ORs the status words of the kernels with bounded waits into one word, in stream order.
__global__ void status_gather_kernel(const unsigned int* a, const unsigned int* b, const unsigned int* c, const unsigned int* d,
                                     const unsigned int* e, unsigned int* out)
{
    out[0] = a[0] | b[0] | c[0] | d[0] | e[0];
}

int gemm(const onn_gemm_args& g, cudaStream_t stream)
{
    ONN_CHECK_ARG(g.A && g.B && g.C);
    ONN_CHECK_ARG(g.M > 0 && g.N > 0 && g.K > 0);
    ONN_CHECK_ARG(g.batch_inner >= 1 && g.batch_outer >= 1);
    ONN_CHECK_ARG((g.a_major == 0 || g.a_major == 1) && (g.b_major == 0 || g.b_major == 1));
    ONN_CHECK_ARG(g.lda >= (g.a_major == 0 ? g.K : g.M));
    ONN_CHECK_ARG(g.ldb >= (g.b_major == 0 ? g.K : g.N));
    ONN_CHECK_ARG(g.ldc >= g.N);
    // split-K partial sums are added atomically: a nonlinear epilogue cannot follow
    ONN_CHECK_ARG(g.split_k <= 1 || (!g.relu && !g.relu_mask && !g.colsum_out && !g.relu_bits && !g.relu_bits_out));
    if(g.relu_bits || g.relu_bits_out)
    {
        ONN_CHECK_ARG(g.batch_inner == 1 && g.batch_outer == 1 && g.relu_bits_ld >= (g.N + 31) / 32);
        ONN_CHECK_ARG(!(g.relu_bits && g.relu_mask));
        ONN_CHECK_ARG(!(g.relu_bits_out && (g.flags & ONN_ACCUMULATE)));
    }

    const int mode = g_mode.load(std::memory_order_relaxed);
    if(g.k_parts > 1)
    {
        ONN_CHECK_ARG(g.batch_inner == 1 && g.batch_outer == 1 && g.split_k <= 1);
        ONN_CHECK_ARG(!g.relu && !g.relu_mask && !g.relu_bits && !g.relu_bits_out);
        if(mode != 1 && gemm_tc_takes_parts(g)) return gemm_tc_launch(g, stream);
        // anywhere else: one product per operand pair, the later ones added to the first
        onn_gemm_args part = g;
        part.k_parts = 0;
        for(int p = 0; p < g.k_parts; p++)
        {
            part.A = g.A + p * g.a_stride_part;
            part.B = g.B + p * g.b_stride_part;
            if(p > 0) { part.flags |= ONN_ACCUMULATE; part.bias = nullptr; }
            const int status = gemm(part, stream);
            if(status != ONN_OK) return status;
        }
        return ONN_OK;
    }
    if(mode == 0 && gemm_skinny_takes(g)) return gemm_skinny_launch(g, stream);
    const bool tc_ok = gemm_tc_supported(g);
    if(mode == 2 && !tc_ok) return ONN_ERR_UNSUPPORTED;
    if(mode != 1 && tc_ok) return gemm_tc_launch(g, stream);
    return gemm_simt_launch(g, stream);
}

}  // namespace onn

using namespace onn;

extern "C" int onn_gemm(const onn_gemm_args* args, void* stream)
{
    ONN_CHECK_ARG(args);
    return gemm(*args, (cudaStream_t)stream);
}

extern "C" int onn_gemm_set_mode(int mode)
{
    ONN_CHECK_ARG(mode >= 0 && mode <= 2);
    g_mode.store(mode, std::memory_order_relaxed);
    return ONN_OK;
}

extern "C" int onn_set_sm_limit(int sms)
{
    ONN_CHECK_ARG(sms >= 0);
    g_sm_limit.store(sms == 0 || sms > kSmCount ? kSmCount : (sms < 2 ? 2 : sms), std::memory_order_relaxed);
    return ONN_OK;
}

// Stand-in for another library's resident kernel (what NCCL's CTAs are to the persistent kernels here): `sms` CTAs that
// each take an SM's shared memory and spin for a fixed number of cycles.  No waiting on anything: it ends by itself.
__global__ void hold_sms_kernel(long long cycles)
{
    extern __shared__ int held[];
    const long long start = clock64();
    long long now = start;
    while(now - start < cycles) now = clock64();
    if(now == 0) held[0] = 0;
}

extern "C" int onn_selftest_hold_sms(int sms, int64_t cycles, void* stream)
{
    ONN_CHECK_ARG(sms > 0 && sms <= kSmCount && cycles > 0 && cycles <= (1LL << 26));    // at most ~35 ms
    constexpr int kHeldBytes = 200 * 1024;                   // no CTA of the persistent kernels fits beside it
    static PerDeviceBytes configured;
    if(!ensure_dynamic_smem(hold_sms_kernel, configured, kHeldBytes)) return ONN_ERR_CUDA;
    hold_sms_kernel<<<sms, 128, kHeldBytes, (cudaStream_t)stream>>>((long long)cycles);
    count_launch();
    return launch_status();
}

extern "C" int onn_set_dynamic_work(int enabled)
{
    const int previous = g_dynamic_work.exchange(enabled != 0 ? 1 : 0, std::memory_order_relaxed);
    return previous == 1 ? 1 : 0;
}

extern "C" int onn_gemm_device_status(void)
{
    const int gemm_status = gemm_tc_read_status();
    const int attention_status = attention_tc_read_status();
    const int loss_status = ce3d_staged_read_status();
    const int long_status = attention_long_read_status();
    const int kv_status = attention_kv_grad_read_status();
    const int status = gemm_status != ONN_OK ? gemm_status : attention_status != ONN_OK ? attention_status : loss_status != ONN_OK ? loss_status :
                       long_status != ONN_OK ? long_status : kv_status;
    if(status != ONN_OK) reset_work_counters();              // a launch that gave up did not leave its counters at zero
    return status;
}

extern "C" int onn_device_status_gather(uint32_t* device_word, void* stream)
{
    ONN_CHECK_ARG(device_word);
    // the three addresses belong to the current device; looked up per device, once
    static std::mutex lock;
    static const unsigned int* words[kMaxDevices][5] = {};
    int device = 0;
    if(cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return ONN_ERR_CUDA;
    const unsigned int* w[5];
    {
        std::lock_guard<std::mutex> guard(lock);
        if(!words[device][0])
        {
            const unsigned int* found[5] = { gemm_tc_status_word(), attention_tc_status_word(), ce3d_staged_status_word(),
                                             attention_long_status_word(), attention_kv_grad_status_word() };
            for(int i = 0; i < 5; i++) if(!found[i]) return ONN_ERR_CUDA;
            for(int i = 0; i < 5; i++) words[device][i] = found[i];
        }
        for(int i = 0; i < 5; i++) w[i] = words[device][i];
    }
    status_gather_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(w[0], w[1], w[2], w[3], w[4], device_word);
    count_launch();
    return launch_status();
}

extern "C" int onn_selftest_bounded_wait(int* gave_up)
{
    ONN_CHECK_ARG(gave_up);
    return gemm_tc_bounded_wait_selftest(gave_up);
}

extern "C" uint64_t onn_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }
extern "C" void onn_launch_count_add(uint64_t launches) { g_launch_count.fetch_add(launches, std::memory_order_relaxed); }

extern "C" int onn_version(void) { return 100; }

extern "C" const char* onn_status_string(int status)
{
    switch(status)
    {
        case ONN_OK: return "ok";
        case ONN_ERR_INVALID_ARGUMENT: return "invalid argument";
        case ONN_ERR_CUDA: return "CUDA call or kernel launch failed";
        case ONN_ERR_UNSUPPORTED: return "unsupported configuration";
        case ONN_ERR_WORKSPACE: return "workspace missing or too small";
        case ONN_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case ONN_ERR_NCCL: return "NCCL call failed";
        case ONN_ERR_LIMIT: return "size beyond a fixed maximum";
        default: return "unknown status";
    }
}
