// Data-parallel gradient exchange: NCCL all-reduce (sum) of contiguous fp32 slices of the
// gradient arena on a dedicated communication stream, ordered against the compute stream
// with events so that reverse-layer buckets overlap the rest of back-propagation.
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
    int world = 1, rank = 0;
};

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
    ONN_CHECK_ARG(out && host_id128 && world >= 1 && rank >= 0 && rank < world);
    onn_dp_comm* c = new (std::nothrow) onn_dp_comm;
    if(!c) return ONN_ERR_CUDA;
    c->world = world; c->rank = rank;
    ncclUniqueId id;
    std::memcpy(&id, host_id128, sizeof(id));
    if(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
       cudaEventCreateWithFlags(&c->ready, cudaEventDisableTiming) != cudaSuccess ||
       cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming) != cudaSuccess)
    {
        delete c;
        return ONN_ERR_CUDA;
    }
    if(ncclCommInitRank(&c->comm, world, id, rank) != ncclSuccess)
    {
        delete c;
        return ONN_ERR_NCCL;
    }
    *out = c;
    return ONN_OK;
}

extern "C" int onn_dp_allreduce(onn_dp_comm* c, float* buf, int64_t n, void* after_stream)
{
    ONN_CHECK_ARG(c && buf && n > 0);
    if(cudaEventRecord(c->ready, (cudaStream_t)after_stream) != cudaSuccess) return ONN_ERR_CUDA;
    if(cudaStreamWaitEvent(c->stream, c->ready, 0) != cudaSuccess) return ONN_ERR_CUDA;
    if(ncclAllReduce(buf, buf, (size_t)n, ncclFloat, ncclSum, c->comm, c->stream) != ncclSuccess) return ONN_ERR_NCCL;
    return ONN_OK;
}

extern "C" int onn_dp_wait(onn_dp_comm* c, void* stream)
{
    ONN_CHECK_ARG(c);
    if(cudaEventRecord(c->done, c->stream) != cudaSuccess) return ONN_ERR_CUDA;
    if(cudaStreamWaitEvent((cudaStream_t)stream, c->done, 0) != cudaSuccess) return ONN_ERR_CUDA;
    ncclResult_t async = ncclSuccess;
    if(ncclCommGetAsyncError(c->comm, &async) != ncclSuccess || async != ncclSuccess) return ONN_ERR_NCCL;
    return ONN_OK;
}

extern "C" int onn_dp_finalize(onn_dp_comm* c)
{
    if(!c) return ONN_OK;
    if(c->stream) cudaStreamSynchronize(c->stream);
    if(c->comm) ncclCommDestroy(c->comm);
    if(c->ready) cudaEventDestroy(c->ready);
    if(c->done) cudaEventDestroy(c->done);
    if(c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return ONN_OK;
}
