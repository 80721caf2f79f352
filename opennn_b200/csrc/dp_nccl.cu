// Data-parallel gradient exchange: NCCL collectives (all-reduce, reduce-scatter, all-gather; sum, fp32) on
// contiguous slices of the gradient and parameter arenas, on a dedicated communication stream that is ordered
// against the compute stream with events, so that reverse-layer buckets overlap the rest of back-propagation.
// NCCL lands peer data in this GPU's own memory; no kernel of this library reads a peer's memory.
#include <nccl.h>

#include <cstring>
#include <new>

#include "common.cuh"

struct onn_dp_comm
{
    ncclComm_t comm = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t ready = nullptr;      // compute -> comm
    cudaEvent_t done = nullptr;       // comm -> compute
    cudaEvent_t marks[ONN_DP_MARKS] = {};   // comm -> compute, one per position a caller wants to wait for separately (made on first use)
    int world = 1, rank = 0;
    bool failed = false;              // a collective failed: the ranks no longer agree on what comes next, so nothing more is enqueued
};

static int after(onn_dp_comm* c, void* stream)
{
    if(c->failed) return ONN_ERR_NCCL;
    if(cudaEventRecord(c->ready, (cudaStream_t)stream) != cudaSuccess) return ONN_ERR_CUDA;
    if(cudaStreamWaitEvent(c->stream, c->ready, 0) != cudaSuccess) return ONN_ERR_CUDA;
    return ONN_OK;
}

static int collective_status(onn_dp_comm* c, ncclResult_t result)
{
    if(result == ncclSuccess) return ONN_OK;
    c->failed = true;
    return ONN_ERR_NCCL;
}

static_assert(sizeof(ncclUniqueId) == 128, "the C ABI hands the NCCL unique id around as 128 bytes");

extern "C" int onn_dp_unique_id(void* host_id128)
{
    ONN_CHECK_ARG(host_id128);
    ncclUniqueId id;
    if(ncclGetUniqueId(&id) != ncclSuccess) return ONN_ERR_NCCL;
    std::memcpy(host_id128, &id, sizeof(id));
    return ONN_OK;
}

extern "C" int onn_dp_init(onn_dp_comm** out, const void* host_id128, int world, int rank)
{
    return onn_dp_init_config(out, host_id128, world, rank, 0);
}

extern "C" int onn_dp_init_config(onn_dp_comm** out, const void* host_id128, int world, int rank, int max_ctas)
{
    ONN_CHECK_ARG(out && host_id128 && world >= 1 && rank >= 0 && rank < world && max_ctas >= 0);
    onn_dp_comm* c = new (std::nothrow) onn_dp_comm;
    if(!c) return ONN_ERR_CUDA;
    c->world = world; c->rank = rank;
    ncclUniqueId id;
    std::memcpy(&id, host_id128, sizeof(id));
    if(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
       cudaEventCreateWithFlags(&c->ready, cudaEventDisableTiming) != cudaSuccess ||
       cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming) != cudaSuccess)
    {
        onn_dp_finalize(c);           // destroys whatever was created
        return ONN_ERR_CUDA;
    }
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    if(max_ctas > 0) config.maxCTAs = max_ctas;       // how many SMs NCCL's kernels may take from back-propagation
    if(ncclCommInitRankConfig(&c->comm, world, id, rank, &config) != ncclSuccess)
    {
        c->comm = nullptr;
        onn_dp_finalize(c);
        return ONN_ERR_NCCL;
    }
    *out = c;
    return ONN_OK;
}

extern "C" int onn_dp_world(const onn_dp_comm* c) { return c ? c->world : 0; }
extern "C" int onn_dp_rank(const onn_dp_comm* c) { return c ? c->rank : -1; }

extern "C" int onn_dp_allreduce(onn_dp_comm* c, float* buf, int64_t n, void* after_stream)
{
    ONN_CHECK_ARG(c && buf && n > 0);
    const int ordered = after(c, after_stream);
    if(ordered != ONN_OK) return ordered;
    return collective_status(c, ncclAllReduce(buf, buf, (size_t)n, ncclFloat, ncclSum, c->comm, c->stream));
}

extern "C" int onn_dp_reduce_scatter(onn_dp_comm* c, const float* send, float* recv, int64_t recv_count, void* after_stream)
{
    ONN_CHECK_ARG(c && send && recv && recv_count > 0);
    const int ordered = after(c, after_stream);
    if(ordered != ONN_OK) return ordered;
    return collective_status(c, ncclReduceScatter(send, recv, (size_t)recv_count, ncclFloat, ncclSum, c->comm, c->stream));
}

extern "C" int onn_dp_all_gather(onn_dp_comm* c, const float* send, float* recv, int64_t send_count, void* after_stream)
{
    ONN_CHECK_ARG(c && send && recv && send_count > 0);
    const int ordered = after(c, after_stream);
    if(ordered != ONN_OK) return ordered;
    return collective_status(c, ncclAllGather(send, recv, (size_t)send_count, ncclFloat, c->comm, c->stream));
}

extern "C" int onn_dp_zero(onn_dp_comm* c, float* buf, int64_t n)
{
    ONN_CHECK_ARG(c && buf && n > 0);
    if(c->failed) return ONN_ERR_NCCL;
    return cudaMemsetAsync(buf, 0, (size_t)n * sizeof(float), c->stream) == cudaSuccess ? ONN_OK : ONN_ERR_CUDA;
}

extern "C" int onn_dp_wait(onn_dp_comm* c, void* stream)
{
    ONN_CHECK_ARG(c);
    if(c->failed) return ONN_ERR_NCCL;
    if(cudaEventRecord(c->done, c->stream) != cudaSuccess) return ONN_ERR_CUDA;
    if(cudaStreamWaitEvent((cudaStream_t)stream, c->done, 0) != cudaSuccess) return ONN_ERR_CUDA;
    ncclResult_t async = ncclSuccess;
    if(ncclCommGetAsyncError(c->comm, &async) != ncclSuccess || async != ncclSuccess) { c->failed = true; return ONN_ERR_NCCL; }
    return ONN_OK;
}

extern "C" int onn_dp_mark(onn_dp_comm* c, int slot)
{
    ONN_CHECK_ARG(c && slot >= 0 && slot < ONN_DP_MARKS);
    if(c->failed) return ONN_ERR_NCCL;
    if(!c->marks[slot] && cudaEventCreateWithFlags(&c->marks[slot], cudaEventDisableTiming) != cudaSuccess) return ONN_ERR_CUDA;
    return cudaEventRecord(c->marks[slot], c->stream) == cudaSuccess ? ONN_OK : ONN_ERR_CUDA;
}

extern "C" int onn_dp_wait_mark(onn_dp_comm* c, int slot, void* stream)
{
    ONN_CHECK_ARG(c && slot >= 0 && slot < ONN_DP_MARKS && c->marks[slot]);
    if(c->failed) return ONN_ERR_NCCL;
    return cudaStreamWaitEvent((cudaStream_t)stream, c->marks[slot], 0) == cudaSuccess ? ONN_OK : ONN_ERR_CUDA;
}

extern "C" int onn_dp_mark_failed(onn_dp_comm* c)
{
    ONN_CHECK_ARG(c);
    c->failed = true;
    return ONN_OK;
}

extern "C" int onn_dp_finalize(onn_dp_comm* c)
{
    if(!c) return ONN_OK;
    if(c->stream) cudaStreamSynchronize(c->stream);
    if(c->comm) ncclCommDestroy(c->comm);
    if(c->ready) cudaEventDestroy(c->ready);
    if(c->done) cudaEventDestroy(c->done);
    for(cudaEvent_t mark : c->marks) if(mark) cudaEventDestroy(mark);
    if(c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return ONN_OK;
}
