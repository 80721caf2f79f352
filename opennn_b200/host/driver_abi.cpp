// C driver ABI over the host mirror (include/onn_b200_host.h): builds a network with its
// loss and optimiser and runs the body of OpenNN's training loop
// (opennn/adaptive_moment_estimation.cpp:697-718) one optimiser step at a time, in
// micro-batches, optionally data-parallel with bucketed gradient all-reduces that overlap
// the rest of back-propagation.
#include <algorithm>
#include <cmath>
#include <cstring>

#include "../../include/onn_b200_host.h"
#include <cstdlib>

#include "opennn_b200.h"

using namespace opennn_b200;

static thread_local string g_last_error;

// An error that keeps its status code across the C boundary (anything else becomes ONN_ERR_CUDA).
struct StatusError : std::runtime_error
{
    StatusError(int status, const string& what) : std::runtime_error(what), status(status) {}
    int status;
};

constexpr Index kMaxMicroBatches = 64;    // statistics slots of one step (BackPropagationCuda::statistics)

struct onn_trainer
{
    unique_ptr<NeuralNetwork> network;
    unique_ptr<CrossEntropyError3d> loss;
    unique_ptr<AdaptiveMomentEstimation> adam;
    unique_ptr<ForwardPropagationCuda> forward;
    unique_ptr<BackPropagationCuda> back;
    unique_ptr<ADAMOptimizationDataCuda> optimization;
    unique_ptr<IncrementalDecoder> decoder;             // created by the first cached decode

    bool decoder_only = false;
    Index micro_batch = 0, input_sequence_length = 0, decoder_sequence_length = 0, vocabulary_size = 0;
    cudaStream_t stream = nullptr;
    bool gradients_dirty = false;

    onn_dp_comm* comm = nullptr;
    int world = 1, rank = 0;
    vector<Index> layer_offsets;          // start of each layer's slice in the gradient arena
    Index pending_high = 0;               // end of the slice not yet handed to the all-reduce
    Index bucket_floats = 16 << 20;       // 64 MiB buckets: large enough for NVLink bandwidth, small enough to overlap

    // Sharded update (data-parallel steps that update): the arena, rounded up to a multiple of 4 * world floats, is cut
    // into buckets of shard_bucket floats on a fixed grid; each bucket is reduce-scattered as soon as back-propagation
    // has finished every gradient in it, rank r receiving the r-th part of each bucket into own_gradient (bucket k's
    // part at k * shard_bucket / world).  The norm is taken over the own parts and summed over ranks, clip + Adam run
    // on the own parts only (moments own_m, own_v: 1 / world of the arena), and an all-gather per bucket brings the
    // updated parameters back to every replica.
    bool sharded_update = true;           // ONN_B200_DP_SHARDED=0: all-reduce + the whole update on every rank
    Index shard_bucket = 0, shard_total = 0, own_size = 0;
    Index pending_bucket = -1;            // highest bucket not yet handed to the reduce-scatter
    bool sharded_step = false;            // this step reduce-scatters (set per step: update and world > 1)
    TensorCuda own_gradient, own_m, own_v;

    // The all-gathers of a sharded update are not waited for at the end of the step: each bucket's gather is marked on
    // the communication stream, and whoever reads parameters next waits for the marks it needs -- the next step's first
    // forward pass layer by layer (so the gathers run under it), every other entry point for all of them.
    bool defer_gather = true;             // ONN_B200_DP_DEFER_GATHER=0: wait at the end of the step
    bool gather_in_flight = false;
    Index gather_buckets = 0;             // buckets of the update whose gathers are in flight
    Index awaited_bucket = -1;            // highest bucket the compute stream already waits for

    // Phase tracing (ONN_B200_TRACE_PHASES=1 or onn_trainer_trace_phases): events on the compute stream at the start
    // of a step, after the last micro-batch's forward pass, after its back-propagation and after the update
    bool trace_phases = false;
    cudaEvent_t phase_events[4] = {};
    bool phases_recorded = false;

    // SMs left to NCCL while a bucket is in flight: the persistent kernels of the next carve_launches launches (rounded
    // up to a layer) occupy 148 - carve_sms SMs, so NCCL's CTAs start at once instead of at a kernel boundary
    int carve_sms = 0, carve_launches = 4;
    bool narrowed = false;
    uint64_t narrowed_at = 0;

    // failure detection in stream order: OR of the kernels' bounded-wait status words, gathered after back-propagation,
    // guards the update and is copied to pinned memory with every step
    TensorCuda status_word;
    volatile uint32_t* pinned_status = nullptr;

    TensorCuda staged_decoder, staged_encoder, staged_targets;

    // int32 feed (onn_trainer_step_host_i32): two sets of device buffers filled by a copy stream, so the ids of the
    // next step cross PCIe while this step computes
    struct IdBuffers { int32_t *decoder = nullptr, *encoder = nullptr, *targets = nullptr; Index capacity = 0;
                       cudaEvent_t copied = nullptr, consumed = nullptr; };
    IdBuffers id_buffers[2];
    cudaStream_t copy_stream = nullptr;
    int id_flip = 0;
    type* pinned_scalars = nullptr;       // {square norm, global active tokens}

    // CUDA-graph replay of the micro-batch: one executable graph per micro-batch index (the statistics slot the
    // loss kernel writes is part of the captured arguments), ids read from fixed buffers
    struct MicroGraph { cudaGraphExec_t executable = nullptr; uint64_t launches = 0; };
    vector<MicroGraph> micro_graphs;
    TensorCuda micro_decoder, micro_encoder, micro_targets;
    bool graphs_enabled = true;
    Index eager_steps = 0;                // graphs are captured only after one eager step has configured every kernel

    // The micro-batch that hands gradient buckets to the exchange cannot be ONE graph: between its kernels the host
    // enqueues collectives on the communication stream and makes the compute stream wait for marks recorded there.  It
    // is replayed as a chain of graph segments instead, cut wherever such an action happens; the actions themselves run
    // between the segments as they do in an eager step.
    struct ExchangeAction { int kind; Index argument; };   // 0: wait for parameter bucket, 1: end of forward pass (all parameters, active-token count), 2: reduce-scatter bucket, -1: none
    struct SegmentedGraph
    {
        vector<cudaGraphExec_t> segments;
        vector<ExchangeAction> actions;                     // actions[i] follows segments[i]
        uint64_t launches = 0;
        Index chunk = -1;                                   // micro-batch number it was recorded for (its statistics slot is a captured argument)
        bool failed = false;
    };
    SegmentedGraph exchange_graph;                          // the micro-batch that hands out the gradient buckets (the last one)
    SegmentedGraph first_graph;                             // the first micro-batch of a step when it is not also the last: waits for parameter buckets only
    SegmentedGraph* recording_graph = nullptr;              // where cut_segment puts what it ends
    bool recording = false;                                 // hooks cut segments instead of acting
    Index recorded_bucket = -1;                             // highest parameter bucket a recorded wait covers

    // cached greedy decoding: one executable graph per target position (the position is part of the captured pointers
    // and arguments), captured from the second call on; ids and END flags live in buffers that never move
    vector<cudaGraphExec_t> decode_graphs;
    vector<uint64_t> decode_graph_launches;
    TensorCuda decode_ids, decode_finished;
    Index cached_decodes = 0;
    int decode_end_id = -1;               // the END id the graphs were captured with (it is a captured argument)

    ~onn_trainer()
    {
        for(MicroGraph& g : micro_graphs) if(g.executable) cudaGraphExecDestroy(g.executable);
        for(cudaGraphExec_t g : exchange_graph.segments) if(g) cudaGraphExecDestroy(g);
        for(cudaGraphExec_t g : first_graph.segments) if(g) cudaGraphExecDestroy(g);
        for(cudaGraphExec_t g : decode_graphs) if(g) cudaGraphExecDestroy(g);
        for(IdBuffers& b : id_buffers)
        {
            if(b.decoder) cudaFree(b.decoder);
            if(b.encoder) cudaFree(b.encoder);
            if(b.targets) cudaFree(b.targets);
            if(b.copied) cudaEventDestroy(b.copied);
            if(b.consumed) cudaEventDestroy(b.consumed);
        }
        for(cudaEvent_t e : phase_events) if(e) cudaEventDestroy(e);
        if(copy_stream) cudaStreamDestroy(copy_stream);
        if(pinned_scalars) cudaFreeHost(pinned_scalars);
        if(pinned_status) cudaFreeHost(const_cast<uint32_t*>(pinned_status));
        if(stream) cudaStreamDestroy(stream);
    }
};

template <typename F>
static int guarded(F&& body)
{
    try { body(); return ONN_OK; }
    catch(const StatusError& e) { g_last_error = e.what(); return e.status; }
    catch(const std::exception& e) { g_last_error = e.what(); return ONN_ERR_CUDA; }
    catch(...) { g_last_error = "unknown exception"; return ONN_ERR_CUDA; }
}

static int environment_int(const char* name, int fallback)
{
    const char* e = std::getenv(name);
    return e && *e ? std::atoi(e) : fallback;
}

// Throws if a kernel of a step already run gave up on a bounded wait (the guarded update of that step did not run).
static void check_device_status(onn_trainer* t)
{
    if(!t->pinned_status || *t->pinned_status == 0) return;
    *t->pinned_status = 0;
    onn_gemm_device_status();                                   // reads and clears the words (synchronises the device)
    if(t->comm) onn_dp_mark_failed(t->comm);                    // this replica skipped an update the others made
    throw StatusError(ONN_ERR_DEVICE_TIMEOUT, "a kernel gave up on a bounded device-side wait; the step's update was skipped");
}

extern "C" const char* onn_trainer_last_error(void) { return g_last_error.c_str(); }

static void await_parameters(onn_trainer* t);
static void settle_parameters(onn_trainer* t);
static void cut_segment(onn_trainer* t, int kind, Index argument);

extern "C" int onn_trainer_create(onn_trainer** out, int network_kind,
                                  int64_t input_sequence_length, int64_t decoder_sequence_length,
                                  int64_t input_vocabulary_size, int64_t output_vocabulary_size,
                                  int64_t embedding_dimension, int64_t heads_number,
                                  int64_t feed_forward_dimension, int64_t layers_number, int64_t micro_batch)
{
    if(!out || micro_batch <= 0) { g_last_error = "onn_trainer_create: bad arguments"; return ONN_ERR_INVALID_ARGUMENT; }
    *out = nullptr;
    return guarded([&]
    {
        int devices = 0;
        if(cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0)
            throw std::runtime_error("no CUDA device: this library has no CPU path");
        auto t = std::make_unique<onn_trainer>();
        check_cuda(cudaStreamCreateWithFlags(&t->stream, cudaStreamNonBlocking), "stream");
        Device::instance().set_compute_stream(t->stream);
        t->decoder_only = network_kind == ONN_NETWORK_DECODER_ONLY;
        t->micro_batch = micro_batch;
        t->input_sequence_length = input_sequence_length;
        t->decoder_sequence_length = decoder_sequence_length;
        t->vocabulary_size = output_vocabulary_size;
        if(t->decoder_only)
            t->network = make_decoder_only_network(decoder_sequence_length, output_vocabulary_size, embedding_dimension, heads_number,
                                                   feed_forward_dimension, layers_number);
        else
            t->network = std::make_unique<Transformer>(input_sequence_length, decoder_sequence_length, input_vocabulary_size,
                                                       output_vocabulary_size, embedding_dimension, heads_number,
                                                       feed_forward_dimension, layers_number);
        t->loss = std::make_unique<CrossEntropyError3d>(t->network.get());
        t->loss->set_regularization_method("None");
        t->adam = std::make_unique<AdaptiveMomentEstimation>(t->loss.get());
        t->forward = std::make_unique<ForwardPropagationCuda>(micro_batch, t->network.get());
        t->back = std::make_unique<BackPropagationCuda>(micro_batch, t->loss.get(), t->forward.get());
        t->optimization = std::make_unique<ADAMOptimizationDataCuda>(t->adam.get());
        if(const char* e = std::getenv("ONN_B200_GRAPHS")) t->graphs_enabled = e[0] != '0';
        check_cuda(cudaMallocHost(reinterpret_cast<void**>(&t->pinned_scalars), 8 * sizeof(type)), "pinned scalars");
        uint32_t* pinned_status = nullptr;
        check_cuda(cudaMallocHost(reinterpret_cast<void**>(&pinned_status), 8 * sizeof(uint32_t)), "pinned status");
        *pinned_status = 0;
        t->pinned_status = pinned_status;
        t->status_word.resize(8);
        t->adam->set_skip_word(reinterpret_cast<const uint32_t*>(t->status_word.data));
        t->sharded_update = environment_int("ONN_B200_DP_SHARDED", 1) != 0;
        t->defer_gather = environment_int("ONN_B200_DP_DEFER_GATHER", 1) != 0;
        t->trace_phases = environment_int("ONN_B200_TRACE_PHASES", 0) != 0;
        t->carve_sms = environment_int("ONN_B200_DP_CARVE_SMS", 0);
        t->carve_launches = environment_int("ONN_B200_DP_CARVE_LAUNCHES", 4);
        t->bucket_floats = std::max(1024, environment_int("ONN_B200_DP_BUCKET_FLOATS", 16 << 20));

        Index offset = 0;
        for(const unique_ptr<Layer>& layer : t->network->get_layers())
        {
            t->layer_offsets.push_back(offset);
            offset += layer->get_parameters_number();
        }
        *out = t.release();
    });
}

extern "C" void onn_trainer_destroy(onn_trainer* trainer)
{
    // no collective may still be writing the parameter arena when it is freed (the communicator is the caller's and may
    // be gone already, so this does not go through it)
    if(trainer && trainer->gather_in_flight) cudaDeviceSynchronize();
    delete trainer;
}

extern "C" int64_t onn_trainer_parameters_number(const onn_trainer* t) { return t ? t->network->get_parameters_number() : 0; }
extern "C" int onn_trainer_layers_number(const onn_trainer* t) { return t ? int(t->network->get_layers_number()) : 0; }

extern "C" int onn_trainer_layer_info(const onn_trainer* t, int layer, char* name, char* label, int capacity,
                                      int64_t* parameters, int64_t* output_size)
{
    if(!t || layer < 0 || layer >= int(t->network->get_layers_number())) return ONN_ERR_INVALID_ARGUMENT;
    Layer* l = t->network->get_layers()[size_t(layer)].get();
    if(name && capacity > 0) { std::strncpy(name, l->get_name().c_str(), size_t(capacity) - 1); name[capacity - 1] = 0; }
    if(label && capacity > 0) { std::strncpy(label, l->get_label().c_str(), size_t(capacity) - 1); label[capacity - 1] = 0; }
    if(parameters) *parameters = l->get_parameters_number();
    if(output_size) *output_size = t->forward->layers[size_t(layer)]->outputs.size();
    return ONN_OK;
}

extern "C" int onn_trainer_set_parameters(onn_trainer* t, const float* host_parameters)
{
    if(!t || !host_parameters) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        settle_parameters(t);
        vector<type>& parameters = t->network->get_parameters();
        std::memcpy(parameters.data(), host_parameters, parameters.size() * sizeof(type));
        t->network->copy_parameters_device();
    });
}

extern "C" int onn_trainer_get_parameters(onn_trainer* t, float* host_parameters)
{
    if(!t || !host_parameters) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        settle_parameters(t);
        t->network->copy_parameters_host();
        const vector<type>& parameters = t->network->get_parameters();
        std::memcpy(host_parameters, parameters.data(), parameters.size() * sizeof(type));
    });
}

extern "C" int onn_trainer_get_gradients(onn_trainer* t, float* host_gradients)
{
    if(!t || !host_gradients) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        check_cuda(cudaStreamSynchronize(t->stream), "synchronize");
        TensorCuda& gradients = t->back->neural_network.gradients;
        check_cuda(cudaMemcpy(host_gradients, gradients.data, size_t(gradients.size()) * sizeof(type), cudaMemcpyDeviceToHost), "get_gradients");
    });
}

extern "C" int onn_trainer_set_learning_rate(onn_trainer* t, float learning_rate)
{
    if(!t) return ONN_ERR_INVALID_ARGUMENT;
    t->adam->set_learning_rate(learning_rate);
    return ONN_OK;
}

extern "C" int onn_trainer_set_iteration(onn_trainer* t, int64_t iteration)
{
    if(!t) return ONN_ERR_INVALID_ARGUMENT;
    t->optimization->iteration = iteration;
    return ONN_OK;
}

extern "C" int onn_trainer_set_dp(onn_trainer* t, onn_dp_comm* comm, int world)
{
    if(!t || world < 1 || (world > 1 && !comm)) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        // gathers of the old communicator and layout: the old communicator is the caller's and may be gone already
        if(t->gather_in_flight) check_cuda(cudaDeviceSynchronize(), "set_dp");
        t->gather_in_flight = false;
        // the recorded exchange belongs to the old communicator and bucket grid
        for(cudaGraphExec_t g : t->exchange_graph.segments) if(g) cudaGraphExecDestroy(g);
        for(cudaGraphExec_t g : t->first_graph.segments) if(g) cudaGraphExecDestroy(g);
        t->exchange_graph = onn_trainer::SegmentedGraph();
        t->first_graph = onn_trainer::SegmentedGraph();
        t->comm = world > 1 ? comm : nullptr;
        t->world = world;
        // NCCL's kernels hold SMs while back-propagation and the next forward pass run: CTAs that start late must not own
        // a fixed share of a launch
        onn_set_dynamic_work(world > 1 ? 1 : 0);
        t->rank = t->comm ? onn_dp_rank(comm) : 0;
        if(t->comm && onn_dp_world(comm) != world) throw std::runtime_error("set_dp: the communicator has another number of ranks");
        t->shard_total = 0;
        const Index parameters_number = t->network->get_parameters_number();
        if(!t->comm || !t->sharded_update)
        {
            // the whole update on this rank: it needs moments for the whole arena
            if(t->optimization->gradient_exponential_decay.size() == 0)
            {
                t->optimization->gradient_exponential_decay.resize(parameters_number);
                t->optimization->square_gradient_exponential_decay.resize(parameters_number);
            }
            t->own_gradient.free(); t->own_m.free(); t->own_v.free();
            return;
        }
        const Index unit = 4 * Index(world);                    // every rank's part of every bucket starts 16-byte aligned
        const Index parameters = t->network->get_parameters_number();
        const Index total = (parameters + unit - 1) / unit * unit;
        if(total > t->back->neural_network.gradients.capacity || total > t->network->get_parameters_device().capacity)
            throw std::runtime_error("set_dp: too many ranks for the sharded update (the arenas are padded to 1024 floats)");
        t->shard_total = total;
        t->shard_bucket = std::max<Index>(unit, t->bucket_floats / unit * unit);
        t->own_size = total / world;
        t->own_gradient.resize(t->own_size);
        t->own_m.resize(t->own_size);
        t->own_v.resize(t->own_size);
        // moments live for the own parts only: 1 / world of the arena each
        t->optimization->gradient_exponential_decay.free();
        t->optimization->square_gradient_exponential_decay.free();
        check_cuda(cudaStreamSynchronize(t->stream), "set_dp");
    });
}

extern "C" int onn_trainer_set_dp_options(onn_trainer* t, int sharded_update, int carve_sms, int carve_launches, int64_t bucket_floats)
{
    if(!t || carve_sms < 0 || carve_launches < 0 || bucket_floats < 0) return ONN_ERR_INVALID_ARGUMENT;
    if(t->comm) { g_last_error = "set_dp_options: call before onn_trainer_set_dp"; return ONN_ERR_INVALID_ARGUMENT; }
    t->sharded_update = sharded_update != 0;
    t->carve_sms = carve_sms;
    t->carve_launches = carve_launches;
    if(bucket_floats > 0) t->bucket_floats = bucket_floats;
    return ONN_OK;
}

static void record_phase(onn_trainer* t, int phase)
{
    if(!t->trace_phases) return;
    if(!t->phase_events[phase]) check_cuda(cudaEventCreate(&t->phase_events[phase]), "phase event");
    check_cuda(cudaEventRecord(t->phase_events[phase], t->stream), "phase event");
    if(phase == 0) t->phases_recorded = false;
    if(phase == 3) t->phases_recorded = true;
}

static int mark_of_bucket(Index bucket) { return int(std::min<Index>(bucket, ONN_DP_MARKS - 1)); }

// The compute stream waits for every parameter all-gather still in flight.
static void await_parameters(onn_trainer* t)
{
    if(!t->gather_in_flight) return;
    t->gather_in_flight = false;
    if(t->awaited_bucket < t->gather_buckets - 1)
        check_onn(onn_dp_wait_mark(t->comm, mark_of_bucket(t->gather_buckets - 1), t->stream), "parameter wait");
    t->awaited_bucket = t->gather_buckets - 1;
}

// ... and for a host-side reader or writer of the parameters: nothing of the update is in flight any more
static void settle_parameters(onn_trainer* t)
{
    await_parameters(t);
    check_cuda(cudaStreamSynchronize(t->stream), "synchronize");
}

// before_layer_hook of the first forward pass after a sharded update: wait for the bucket that holds the END of this
// layer's parameters (the communication stream runs in order, so the earlier buckets are then complete too)
static void await_layer_parameters(void* context, Index layer)
{
    onn_trainer* t = static_cast<onn_trainer*>(context);
    if(!t->gather_in_flight && !t->recording) return;
    const Index low = t->layer_offsets[size_t(layer)];
    const Index high = size_t(layer) + 1 < t->layer_offsets.size() ? t->layer_offsets[size_t(layer) + 1] : t->network->get_parameters_number();
    if(high <= low) return;
    if(t->recording)
    {
        // every replay may find gathers in flight: cut wherever a layer's parameters end in a bucket no earlier wait covers
        const Index bucket = (high - 1) / t->shard_bucket;
        if(bucket > t->recorded_bucket) { cut_segment(t, 0, bucket); t->recorded_bucket = bucket; }
        return;
    }
    const Index needed = std::min((high - 1) / t->shard_bucket, t->gather_buckets - 1);
    if(needed <= t->awaited_bucket) return;
    check_onn(onn_dp_wait_mark(t->comm, mark_of_bucket(needed), t->stream), "parameter wait");
    t->awaited_bucket = needed;
    if(needed == t->gather_buckets - 1) t->gather_in_flight = false;
}

static void narrow_for_exchange(onn_trainer* t)
{
    if(t->carve_sms <= 0) return;
    check_onn(onn_set_sm_limit(148 - t->carve_sms), "sm limit");
    t->narrowed = true;
    t->narrowed_at = onn_launch_count();
}

static void widen_after_exchange(onn_trainer* t, bool now)
{
    if(!t->narrowed) return;
    if(!now && onn_launch_count() - t->narrowed_at < uint64_t(t->carve_launches)) return;
    onn_set_sm_limit(0);
    t->narrowed = false;
}

// Bucket k of the fixed grid: reduce-scatter into the own parts, then clear it for the next step off the compute stream.
static void reduce_scatter_bucket(onn_trainer* t, Index k)
{
    const Index low = k * t->shard_bucket;
    const Index size = std::min(t->shard_bucket, t->shard_total - low);
    type* gradients = t->back->neural_network.gradients.data;
    check_onn(onn_dp_reduce_scatter(t->comm, gradients + low, t->own_gradient.data + low / t->world, size / t->world, t->stream),
              "gradient reduce-scatter");
    check_onn(onn_dp_zero(t->comm, gradients + low, size), "gradient bucket clear");
}

// Called after layer `layer` has back-propagated: every gradient slice from this layer's offset up is final on the
// compute stream.  Hands what is complete to the exchange: whole buckets of the fixed grid (sharded update) or the
// layers gathered so far once they make up a bucket (all-reduce).  layer < 0: everything that is left.
static void gradient_ready(void* context, Index layer)
{
    onn_trainer* t = static_cast<onn_trainer*>(context);
    const Index low = layer <= 0 ? 0 : t->layer_offsets[size_t(layer)];
    bool issued = false;
    if(t->sharded_step)
    {
        for(; t->pending_bucket >= 0 && t->pending_bucket * t->shard_bucket >= low; t->pending_bucket--)
        {
            if(t->recording) { cut_segment(t, 2, t->pending_bucket); continue; }
            if(!issued) narrow_for_exchange(t);
            issued = true;
            reduce_scatter_bucket(t, t->pending_bucket);
        }
    }
    else if(t->pending_high - low >= t->bucket_floats || (layer <= 0 && t->pending_high > low))
    {
        narrow_for_exchange(t);
        issued = true;
        check_onn(onn_dp_allreduce(t->comm, t->back->neural_network.gradients.data + low, t->pending_high - low, t->stream),
                  "gradient all-reduce");
        t->pending_high = low;
    }
    if(!issued) widen_after_exchange(t, false);
}

// Clip + Adam on this rank's parts of the reduced gradient, then the updated parameters back to every replica.
static void sharded_update(onn_trainer* t)
{
    check_onn(onn_dp_wait(t->comm, t->stream), "gradient wait");
    type* square_norm = t->optimization->square_norm.data;
    check_onn(onn_grad_sqnorm(t->own_gradient.data, t->own_size, square_norm, t->optimization->norm_workspace.data, t->stream), "gradient norm");
    check_onn(onn_dp_allreduce(t->comm, square_norm, 1, t->stream), "gradient norm all-reduce");
    check_onn(onn_dp_wait(t->comm, t->stream), "gradient norm wait");

    type bias_correction_1, bias_correction_2;
    t->adam->advance(*t->optimization, bias_correction_1, bias_correction_2);
    type* parameters = t->network->get_parameters_device().data;
    const uint32_t* skip = reinterpret_cast<const uint32_t*>(t->status_word.data);
    const Index buckets = (t->shard_total + t->shard_bucket - 1) / t->shard_bucket;
    for(Index k = 0; k < buckets; k++)
    {
        const Index low = k * t->shard_bucket;
        const Index part = std::min(t->shard_bucket, t->shard_total - low) / t->world;
        type* own_parameters = parameters + low + t->rank * part;
        const Index own = low / t->world;
        check_onn(onn_adam_guarded(own_parameters, t->own_m.data + own, t->own_v.data + own, t->own_gradient.data + own, part,
                                   t->adam->get_learning_rate(), t->adam->get_beta_1(), t->adam->get_beta_2(), EPSILON,
                                   bias_correction_1, bias_correction_2, t->adam->get_gradient_clip_norm(), square_norm, type(1), 0, skip,
                                   t->stream), "sharded Adam");
        // the all-gather of this bucket waits for this bucket's update only and overlaps the next bucket's
        check_onn(onn_dp_all_gather(t->comm, own_parameters, parameters + low, part, t->stream), "parameter all-gather");
        check_onn(onn_dp_mark(t->comm, mark_of_bucket(k)), "parameter mark");
    }
    t->gather_in_flight = true;
    t->gather_buckets = buckets;
    t->awaited_bucket = -1;
    if(!t->defer_gather) await_parameters(t);
}

// Replays (capturing it first if need be) the forward pass, loss and back-propagation of micro-batch number `chunk`.
// Returns false if graphs cannot be used; the caller then runs the micro-batch eagerly.
static bool replay_micro_batch(onn_trainer* t, const BatchCuda& source, Index chunk)
{
    const Index S_dec = t->decoder_sequence_length, S_in = t->input_sequence_length;
    if(t->micro_decoder.size() == 0)
    {
        t->micro_decoder.resize(t->micro_batch * S_dec);
        t->micro_targets.resize(t->micro_batch * S_dec);
        if(!t->decoder_only) t->micro_encoder.resize(t->micro_batch * S_in);
    }
    if(size_t(chunk) >= t->micro_graphs.size()) t->micro_graphs.resize(size_t(chunk) + 1);
    onn_trainer::MicroGraph& graph = t->micro_graphs[size_t(chunk)];

    // the captured kernels read their ids from these fixed buffers
    const size_t decoder_bytes = size_t(t->micro_batch * S_dec) * sizeof(type);
    check_cuda(cudaMemcpyAsync(t->micro_decoder.data, source.decoder.data, decoder_bytes, cudaMemcpyDeviceToDevice, t->stream), "micro ids");
    check_cuda(cudaMemcpyAsync(t->micro_targets.data, source.target.data, decoder_bytes, cudaMemcpyDeviceToDevice, t->stream), "micro targets");
    if(!t->decoder_only)
        check_cuda(cudaMemcpyAsync(t->micro_encoder.data, source.input.data, size_t(t->micro_batch * S_in) * sizeof(type),
                                   cudaMemcpyDeviceToDevice, t->stream), "micro ids");

    if(!graph.executable)
    {
        BatchCuda micro;
        micro.samples_number = t->micro_batch;
        micro.decoder = TensorViewCuda(t->micro_decoder.data, {t->micro_batch, S_dec});
        if(!t->decoder_only) micro.input = TensorViewCuda(t->micro_encoder.data, {t->micro_batch, S_in});
        micro.target = TensorViewCuda(t->micro_targets.data, {t->micro_batch, S_dec});

        const Index slot_before = t->back->statistics_slot;
        const uint64_t launches_before = onn_launch_count();
        cudaGraph_t captured = nullptr;
        bool ok = cudaStreamBeginCapture(t->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if(ok)
        {
            try
            {
                t->network->forward_propagate(micro.get_inputs_device(), *t->forward, true);
                t->loss->back_propagate(micro, *t->forward, *t->back, chunk > 0);
            }
            catch(...) { ok = false; }
            ok = (cudaStreamEndCapture(t->stream, &captured) == cudaSuccess) && ok && captured != nullptr;
        }
        if(ok) ok = cudaGraphInstantiate(&graph.executable, captured, 0) == cudaSuccess;
        if(captured) cudaGraphDestroy(captured);
        if(!ok)
        {
            // nothing of the micro-batch has run; give up on graphs for this trainer and let the caller run it eagerly
            cudaGetLastError();
            graph.executable = nullptr;
            t->graphs_enabled = false;
            t->back->statistics_slot = slot_before;
            return false;
        }
        graph.launches = onn_launch_count() - launches_before;    // counted at capture; the first replay below is that launch
        t->back->statistics_slot = slot_before;
        onn_launch_count_add(0 - graph.launches);
    }

    // host-side bookkeeping the captured code did when it ran eagerly
    if(chunk == 0) t->back->statistics_slot = 0;
    t->back->statistics_slot++;
    check_cuda(cudaGraphLaunch(graph.executable, t->stream), "micro-batch graph launch");
    onn_launch_count_add(graph.launches);
    return true;
}

// What the host does between two segments of the exchanging micro-batch (and what an eager step does at the same place).
static void perform(onn_trainer* t, const onn_trainer::ExchangeAction& action)
{
    switch(action.kind)
    {
        case 0:                                              // the forward pass is about to read parameters up to this bucket
            if(t->gather_in_flight)
            {
                const Index needed = std::min(action.argument, t->gather_buckets - 1);
                if(needed > t->awaited_bucket)
                {
                    check_onn(onn_dp_wait_mark(t->comm, mark_of_bucket(needed), t->stream), "parameter wait");
                    t->awaited_bucket = needed;
                    if(needed == t->gather_buckets - 1) t->gather_in_flight = false;
                }
            }
            break;
        case 1:                                              // forward pass done: the loss reads the global active-token count
            await_parameters(t);
            check_onn(onn_dp_wait(t->comm, t->stream), "active-token wait");
            break;
        case 2:
            reduce_scatter_bucket(t, action.argument);
            break;
        default: break;
    }
}

// Ends the segment being captured, remembers the action that follows it, and starts the next one.
static void cut_segment(onn_trainer* t, int kind, Index argument)
{
    onn_trainer::SegmentedGraph& graph = *t->recording_graph;
    cudaGraph_t captured = nullptr;
    if(cudaStreamEndCapture(t->stream, &captured) != cudaSuccess || !captured) throw std::runtime_error("segment capture failed");
    cudaGraphExec_t executable = nullptr;
    const bool ok = cudaGraphInstantiate(&executable, captured, 0) == cudaSuccess;
    cudaGraphDestroy(captured);
    if(!ok) throw std::runtime_error("segment instantiation failed");
    graph.segments.push_back(executable);
    graph.actions.push_back({kind, argument});
    if(kind >= 0 && cudaStreamBeginCapture(t->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
        throw std::runtime_error("segment capture failed");
}

// Replays (recording it first if need be) a micro-batch in whose middle the host has to act: the one that hands its
// gradient buckets to the reduce-scatter (hands_out), and the first one of a step, whose forward pass waits for the
// parameter gathers of the step before.  Returns false if it cannot be done this way; the caller then runs the
// micro-batch another way.
static bool replay_segmented_micro_batch(onn_trainer* t, onn_trainer::SegmentedGraph& graph, const BatchCuda& source, Index chunk, bool hands_out)
{
    if(graph.failed || (graph.chunk >= 0 && graph.chunk != chunk)) return false;
    const Index S_dec = t->decoder_sequence_length, S_in = t->input_sequence_length;
    if(t->micro_decoder.size() == 0)
    {
        t->micro_decoder.resize(t->micro_batch * S_dec);
        t->micro_targets.resize(t->micro_batch * S_dec);
        if(!t->decoder_only) t->micro_encoder.resize(t->micro_batch * S_in);
    }
    // the captured kernels read their ids from these fixed buffers
    const size_t decoder_bytes = size_t(t->micro_batch * S_dec) * sizeof(type);
    check_cuda(cudaMemcpyAsync(t->micro_decoder.data, source.decoder.data, decoder_bytes, cudaMemcpyDeviceToDevice, t->stream), "micro ids");
    check_cuda(cudaMemcpyAsync(t->micro_targets.data, source.target.data, decoder_bytes, cudaMemcpyDeviceToDevice, t->stream), "micro targets");
    if(!t->decoder_only)
        check_cuda(cudaMemcpyAsync(t->micro_encoder.data, source.input.data, size_t(t->micro_batch * S_in) * sizeof(type),
                                   cudaMemcpyDeviceToDevice, t->stream), "micro ids");

    if(graph.segments.empty())
    {
        BatchCuda micro;
        micro.samples_number = t->micro_batch;
        micro.decoder = TensorViewCuda(t->micro_decoder.data, {t->micro_batch, S_dec});
        if(!t->decoder_only) micro.input = TensorViewCuda(t->micro_encoder.data, {t->micro_batch, S_in});
        micro.target = TensorViewCuda(t->micro_targets.data, {t->micro_batch, S_dec});

        const Index slot_before = t->back->statistics_slot;
        const uint64_t launches_before = onn_launch_count();
        bool ok = cudaStreamBeginCapture(t->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if(ok)
        {
            t->recording = true;
            t->recording_graph = &graph;
            t->recorded_bucket = -1;
            try
            {
                t->network->before_layer_hook = await_layer_parameters;
                t->network->before_layer_context = t;
                t->network->forward_propagate(micro.get_inputs_device(), *t->forward, true);
                t->network->before_layer_hook = nullptr;
                cut_segment(t, 1, 0);
                if(hands_out)
                {
                    t->pending_bucket = (t->shard_total - 1) / t->shard_bucket;
                    t->loss->gradient_ready_hook = gradient_ready;
                    t->loss->gradient_ready_context = t;
                }
                t->loss->back_propagate(micro, *t->forward, *t->back, chunk > 0);
                if(hands_out) gradient_ready(t, -1);
                t->loss->gradient_ready_hook = nullptr;
                cut_segment(t, -1, 0);
            }
            catch(...)
            {
                ok = false;
                cudaGraph_t abandoned = nullptr;
                cudaStreamEndCapture(t->stream, &abandoned);     // leaves capture mode whatever state it is in
                if(abandoned) cudaGraphDestroy(abandoned);
            }
            t->recording = false;
            t->network->before_layer_hook = nullptr;
            t->loss->gradient_ready_hook = nullptr;
        }
        t->back->statistics_slot = slot_before;
        if(!ok)
        {
            // nothing of the micro-batch has run; give up on this way of running it and let the caller run it eagerly
            cudaGetLastError();
            for(cudaGraphExec_t g : graph.segments) if(g) cudaGraphExecDestroy(g);
            graph.segments.clear();
            graph.actions.clear();
            graph.failed = true;
            onn_launch_count_add(0 - (onn_launch_count() - launches_before));
            return false;
        }
        graph.launches = onn_launch_count() - launches_before;    // counted at capture; the replay below is that launch
        graph.chunk = chunk;
        onn_launch_count_add(0 - graph.launches);
    }

    // host-side bookkeeping the captured code did when it ran eagerly
    if(chunk == 0) t->back->statistics_slot = 0;
    t->back->statistics_slot++;
    for(size_t i = 0; i < graph.segments.size(); i++)
    {
        check_cuda(cudaGraphLaunch(graph.segments[i], t->stream), "segment launch");
        perform(t, graph.actions[i]);
    }
    onn_launch_count_add(graph.launches);
    return true;
}

// Whatever ends the step, the hook that hands gradients to the exchange does not outlive it and the SM limit is lifted.
struct ExchangeScope
{
    explicit ExchangeScope(onn_trainer* t) : t(t) {}
    ~ExchangeScope()
    {
        t->loss->gradient_ready_hook = nullptr;
        t->network->before_layer_hook = nullptr;
        widen_after_exchange(t, true);
    }
    onn_trainer* t;
};

static void run_step_body(onn_trainer* t, const float* decoder_ids, const float* encoder_ids, const float* targets,
                          Index batch, bool update, float* statistics);

static void run_step(onn_trainer* t, const float* decoder_ids, const float* encoder_ids, const float* targets,
                     Index batch, bool update, float* statistics)
{
    if(batch <= 0 || batch % t->micro_batch != 0) throw std::runtime_error("step: batch must be a positive multiple of micro_batch");
    if(batch / t->micro_batch > kMaxMicroBatches) throw std::runtime_error("step: at most 64 micro-batches per step (batch / micro_batch)");
    if(!decoder_ids || !targets || (!t->decoder_only && !encoder_ids)) throw std::runtime_error("step: missing ids or targets");
    check_device_status(t);
    try { run_step_body(t, decoder_ids, encoder_ids, targets, batch, update, statistics); }
    catch(...)
    {
        // a step that ends half-way has joined some of its collectives and not others: the ranks no longer agree on
        // which one comes next, so this rank must not enqueue another
        if(t->comm) onn_dp_mark_failed(t->comm);
        throw;
    }
}

static void run_step_body(onn_trainer* t, const float* decoder_ids, const float* encoder_ids, const float* targets,
                          Index batch, bool update, float* statistics)
{
    Device::instance().set_compute_stream(t->stream);
    ExchangeScope scope(t);
    t->sharded_step = t->comm && update && t->shard_total > 0;
    const Index S_dec = t->decoder_sequence_length, S_in = t->input_sequence_length;
    TensorCuda& gradients = t->back->neural_network.gradients;

    record_phase(t, 0);
    if(t->gradients_dirty) gradients.fill(0);                // adaptive_moment_estimation.cpp:699 (Adam leaves them zero otherwise)
    t->gradients_dirty = true;

    // #active over the whole batch (and over all ranks): the loss gradient of every micro-batch is scaled by it
    BatchCuda whole;
    whole.samples_number = batch;
    whole.target = TensorViewCuda(const_cast<float*>(targets), {batch, S_dec});
    t->loss->calculate_active_tokens(whole, *t->back);
    // The count is first read by the loss kernel, so the compute stream waits for it only there: the communication
    // stream may still be busy with the parameter gathers of the previous step, which the forward pass overlaps.
    bool count_pending = false;
    if(t->comm)
    {
        check_onn(onn_dp_allreduce(t->comm, t->back->active_count.data, 1, t->stream), "active-token all-reduce");
        count_pending = true;
    }
    const auto await_count = [&]
    {
        if(!count_pending) return;
        count_pending = false;
        check_onn(onn_dp_wait(t->comm, t->stream), "active-token wait");
    };

    const Index chunks = batch / t->micro_batch;
    for(Index chunk = 0; chunk < chunks; chunk++)
    {
        const Index first = chunk * t->micro_batch;
        BatchCuda micro;
        micro.samples_number = t->micro_batch;
        micro.decoder = TensorViewCuda(const_cast<float*>(decoder_ids) + first * S_dec, {t->micro_batch, S_dec});
        if(!t->decoder_only) micro.input = TensorViewCuda(const_cast<float*>(encoder_ids) + first * S_in, {t->micro_batch, S_in});
        micro.target = TensorViewCuda(const_cast<float*>(targets) + first * S_dec, {t->micro_batch, S_dec});

        const bool last = chunk == chunks - 1;
        const bool hands_out_gradients = t->comm && last;     // bucketed all-reduces are issued from inside back-propagation
        if(t->graphs_enabled && t->eager_steps > 0 && !hands_out_gradients)
        {
            // the first micro-batch after a sharded update: cut where its forward pass meets a parameter bucket the
            // gathers may still be bringing, so that they run under it
            if(chunk == 0 && t->comm && t->sharded_update && t->shard_total > 0 && !t->trace_phases &&
               replay_segmented_micro_batch(t, t->first_graph, micro, chunk, false))
            {
                count_pending = false;
                continue;
            }
            // a micro-batch replayed as one graph cannot wait layer by layer: everything it reads must be there before it starts
            await_parameters(t);
            await_count();
            if(replay_micro_batch(t, micro, chunk)) continue;
        }

        if(hands_out_gradients && t->sharded_step && t->graphs_enabled && t->eager_steps > 0 && !t->trace_phases && t->carve_sms == 0 &&
           replay_segmented_micro_batch(t, t->exchange_graph, micro, chunk, true))
        {
            count_pending = false;                               // waited for between the segments
            continue;
        }

        if(t->gather_in_flight)
        {
            t->network->before_layer_hook = await_layer_parameters;
            t->network->before_layer_context = t;
        }
        t->network->forward_propagate(micro.get_inputs_device(), *t->forward, true);
        t->network->before_layer_hook = nullptr;
        await_parameters(t);                                     // whatever no layer asked for (padding at the end of the arena)
        await_count();
        if(last) record_phase(t, 1);

        if(hands_out_gradients)
        {
            t->pending_high = gradients.size();
            t->pending_bucket = t->sharded_step ? (t->shard_total - 1) / t->shard_bucket : -1;
            t->loss->gradient_ready_hook = gradient_ready;
            t->loss->gradient_ready_context = t;
        }
        t->loss->back_propagate(micro, *t->forward, *t->back, chunk > 0);
        if(hands_out_gradients) gradient_ready(t, -1);           // whatever the layer walk left (it ends at the first trainable layer)
        t->loss->gradient_ready_hook = nullptr;
        widen_after_exchange(t, true);
        if(last) record_phase(t, 2);
    }
    t->eager_steps++;

    // OR of the bounded-wait status words of everything this step has run: guards the update, read with the statistics
    uint32_t* status_word = reinterpret_cast<uint32_t*>(t->status_word.data);
    check_onn(onn_device_status_gather(status_word, t->stream), "device status");

    if(t->comm)
        check_onn(onn_dp_allreduce(t->comm, t->back->statistics.data, 4 * t->back->statistics_slot, t->stream), "statistics all-reduce");

    if(t->sharded_step)
    {
        sharded_update(t);
        t->gradients_dirty = false;                              // every bucket was cleared after its reduce-scatter
    }
    else
    {
        if(t->comm) check_onn(onn_dp_wait(t->comm, t->stream), "gradient wait");
        if(update)
        {
            t->adam->update_parameters(*t->back, *t->optimization);
            t->gradients_dirty = false;                          // the update kernel zeroes the arena for the next step
        }
        else if(statistics)
            check_onn(onn_grad_sqnorm(gradients.data, gradients.size(), t->optimization->square_norm.data, t->optimization->norm_workspace.data,
                                      t->stream), "gradient norm");
    }
    record_phase(t, 3);
    check_cuda(cudaMemcpyAsync(const_cast<uint32_t*>(t->pinned_status), status_word, sizeof(uint32_t), cudaMemcpyDeviceToHost, t->stream), "status readback");

    if(statistics)
    {
        check_cuda(cudaMemcpyAsync(t->pinned_scalars, t->optimization->square_norm.data, sizeof(type), cudaMemcpyDeviceToHost, t->stream), "norm readback");
        check_cuda(cudaMemcpyAsync(t->pinned_scalars + 1, t->back->active_count.data, sizeof(type), cudaMemcpyDeviceToHost, t->stream), "count readback");
        t->loss->read_error(*t->back, 0);                        // synchronises the stream
        check_device_status(t);
        // statistics slots were summed over ranks; so is the active count in pinned_scalars[1]
        double loss_sum = 0, correct = 0;
        for(Index k = 0; k < t->back->statistics_slot; k++)
        {
            loss_sum += t->back->pinned_statistics[4 * k];
            correct += t->back->pinned_statistics[4 * k + 1];
        }
        const double active = t->pinned_scalars[1];
        statistics[0] = active > 0 ? float(loss_sum / active) : 0.f;
        statistics[1] = active > 0 ? float(correct / active) : 0.f;
        statistics[2] = float(active);
        statistics[3] = std::sqrt(t->pinned_scalars[0]);
    }
}

extern "C" int onn_trainer_set_graph_capture(onn_trainer* t, int enabled)
{
    if(!t) return ONN_ERR_INVALID_ARGUMENT;
    t->graphs_enabled = enabled != 0;
    return ONN_OK;
}

extern "C" int onn_trainer_step_device(onn_trainer* t, const float* decoder_ids, const float* encoder_ids, const float* targets,
                                       int64_t batch, int update, float* statistics)
{
    if(!t) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&] { run_step(t, decoder_ids, encoder_ids, targets, batch, update != 0, statistics); });
}

extern "C" int onn_trainer_step_host(onn_trainer* t, const float* decoder_ids, const float* encoder_ids, const float* targets,
                                     int64_t batch, int update, float* statistics)
{
    if(!t || !decoder_ids || !targets) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        const Index decoder_count = batch * t->decoder_sequence_length, encoder_count = batch * t->input_sequence_length;
        if(t->staged_decoder.size() < decoder_count) { t->staged_decoder.resize(decoder_count); t->staged_targets.resize(decoder_count); }
        if(!t->decoder_only && t->staged_encoder.size() < encoder_count) t->staged_encoder.resize(encoder_count);
        check_cuda(cudaMemcpyAsync(t->staged_decoder.data, decoder_ids, size_t(decoder_count) * sizeof(type), cudaMemcpyHostToDevice, t->stream), "ids H2D");
        check_cuda(cudaMemcpyAsync(t->staged_targets.data, targets, size_t(decoder_count) * sizeof(type), cudaMemcpyHostToDevice, t->stream), "targets H2D");
        if(!t->decoder_only)
        {
            if(!encoder_ids) throw std::runtime_error("step: missing encoder ids");
            check_cuda(cudaMemcpyAsync(t->staged_encoder.data, encoder_ids, size_t(encoder_count) * sizeof(type), cudaMemcpyHostToDevice, t->stream), "ids H2D");
        }
        run_step(t, t->staged_decoder.data, t->decoder_only ? nullptr : t->staged_encoder.data, t->staged_targets.data, batch, update != 0, statistics);
    });
}

extern "C" int onn_trainer_step_host_i32(onn_trainer* t, const int32_t* decoder_ids, const int32_t* encoder_ids, const int32_t* targets,
                                         int64_t batch, int update, float* statistics)
{
    if(!t || !decoder_ids || !targets || batch <= 0) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        if(!t->decoder_only && !encoder_ids) throw std::runtime_error("step: missing encoder ids");
        const Index decoder_count = batch * t->decoder_sequence_length, encoder_count = batch * t->input_sequence_length;
        if(!t->copy_stream) check_cuda(cudaStreamCreateWithFlags(&t->copy_stream, cudaStreamNonBlocking), "copy stream");
        onn_trainer::IdBuffers& ids = t->id_buffers[t->id_flip];
        t->id_flip ^= 1;
        const Index wanted = std::max(decoder_count, encoder_count);
        if(ids.capacity < wanted)
        {
            if(ids.copied) check_cuda(cudaEventSynchronize(ids.copied), "id buffers");       // nothing may still use the old ones
            if(ids.consumed) check_cuda(cudaEventSynchronize(ids.consumed), "id buffers");
            for(int32_t** pointer : {&ids.decoder, &ids.encoder, &ids.targets})
            {
                if(*pointer) cudaFree(*pointer);
                check_cuda(cudaMalloc(reinterpret_cast<void**>(pointer), size_t(wanted) * sizeof(int32_t)), "id buffers");
            }
            ids.capacity = wanted;
            if(!ids.copied) check_cuda(cudaEventCreateWithFlags(&ids.copied, cudaEventDisableTiming), "id event");
            if(!ids.consumed) check_cuda(cudaEventCreateWithFlags(&ids.consumed, cudaEventDisableTiming), "id event");
        }
        if(t->staged_decoder.size() < decoder_count) { t->staged_decoder.resize(decoder_count); t->staged_targets.resize(decoder_count); }
        if(!t->decoder_only && t->staged_encoder.size() < encoder_count) t->staged_encoder.resize(encoder_count);

        // copy stream: wait until the conversion kernels that last read this set are done, then bring the new ids over
        check_cuda(cudaStreamWaitEvent(t->copy_stream, ids.consumed, 0), "id buffers: wait for consumer");
        check_cuda(cudaMemcpyAsync(ids.decoder, decoder_ids, size_t(decoder_count) * sizeof(int32_t), cudaMemcpyHostToDevice, t->copy_stream), "ids H2D");
        check_cuda(cudaMemcpyAsync(ids.targets, targets, size_t(decoder_count) * sizeof(int32_t), cudaMemcpyHostToDevice, t->copy_stream), "targets H2D");
        if(!t->decoder_only)
            check_cuda(cudaMemcpyAsync(ids.encoder, encoder_ids, size_t(encoder_count) * sizeof(int32_t), cudaMemcpyHostToDevice, t->copy_stream), "ids H2D");
        check_cuda(cudaEventRecord(ids.copied, t->copy_stream), "id buffers: copied");

        // compute stream: ids as the floats the layers read
        check_cuda(cudaStreamWaitEvent(t->stream, ids.copied, 0), "id buffers: wait for copy");
        check_onn(onn_ids_to_float(ids.decoder, t->staged_decoder.data, decoder_count, t->stream), "ids to float");
        check_onn(onn_ids_to_float(ids.targets, t->staged_targets.data, decoder_count, t->stream), "ids to float");
        if(!t->decoder_only) check_onn(onn_ids_to_float(ids.encoder, t->staged_encoder.data, encoder_count, t->stream), "ids to float");
        check_cuda(cudaEventRecord(ids.consumed, t->stream), "id buffers: consumed");
        run_step(t, t->staged_decoder.data, t->decoder_only ? nullptr : t->staged_encoder.data, t->staged_targets.data, batch, update != 0, statistics);
    });
}

extern "C" int onn_trainer_forward(onn_trainer* t, const float* decoder_ids, const float* encoder_ids, int is_training)
{
    if(!t || !decoder_ids) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        Device::instance().set_compute_stream(t->stream);
        await_parameters(t);
        BatchCuda micro;
        micro.samples_number = t->micro_batch;
        micro.decoder = TensorViewCuda(const_cast<float*>(decoder_ids), {t->micro_batch, t->decoder_sequence_length});
        if(!t->decoder_only) micro.input = TensorViewCuda(const_cast<float*>(encoder_ids), {t->micro_batch, t->input_sequence_length});
        t->network->forward_propagate(micro.get_inputs_device(), *t->forward, is_training != 0);
    });
}

extern "C" int onn_trainer_greedy_decode(onn_trainer* t, const float* encoder_ids, float* decoded_ids, int start_id, int end_id)
{
    if(!t || !encoder_ids || !decoded_ids || t->decoder_only) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        Device::instance().set_compute_stream(t->stream);
        await_parameters(t);
        const Index B = t->micro_batch, S_in = t->input_sequence_length, S_dec = t->decoder_sequence_length;
        if(t->staged_encoder.size() < B * S_in) t->staged_encoder.resize(B * S_in);
        if(t->staged_decoder.size() < B * S_dec) { t->staged_decoder.resize(B * S_dec); t->staged_targets.resize(B * S_dec); }
        TensorCuda finished_device;
        finished_device.resize(B);                                  // zero-filled; read as int

        // target ids start as [START, PAD, ...] (opennn/standard_networks.cpp:1002-1004)
        vector<type> target(size_t(B * S_dec), type(0));
        for(Index b = 0; b < B; b++) target[size_t(b * S_dec)] = type(start_id);
        check_cuda(cudaMemcpyAsync(t->staged_encoder.data, encoder_ids, size_t(B * S_in) * sizeof(type), cudaMemcpyHostToDevice, t->stream), "ids H2D");
        check_cuda(cudaMemcpyAsync(t->staged_decoder.data, target.data(), target.size() * sizeof(type), cudaMemcpyHostToDevice, t->stream), "ids H2D");
        check_cuda(cudaStreamSynchronize(t->stream), "decode: ids");   // `target` is pageable host memory

        BatchCuda batch;
        batch.samples_number = B;
        batch.decoder = TensorViewCuda(t->staged_decoder.data, {B, S_dec});
        batch.input = TensorViewCuda(t->staged_encoder.data, {B, S_in});
        // the reference re-runs the whole network for every token; the encoder side sees the same ids each time, so it
        // runs once here and only the layers that depend on the decoder ids run per token
        const vector<char> decoder_side = t->network->layers_depending_on_input(1);
        vector<int> finished(size_t(B), 0);
        for(Index i = 1; i < S_dec; i++)
        {
            t->network->forward_propagate(batch.get_inputs_device(), *t->forward, false, i == 1 ? nullptr : &decoder_side);
            const TensorViewCuda outputs = t->forward->get_outputs();
            check_onn(onn_greedy_next_token(outputs.data, t->staged_decoder.data, reinterpret_cast<int*>(finished_device.data), B, S_dec,
                                            t->vocabulary_size, i - 1, end_id, t->stream), "greedy step");
            if(i % 8 == 0 || i + 1 == S_dec)
            {
                check_cuda(cudaMemcpyAsync(finished.data(), finished_device.data, size_t(B) * sizeof(int), cudaMemcpyDeviceToHost, t->stream), "decode: flags");
                check_cuda(cudaStreamSynchronize(t->stream), "decode: flags");
                bool all = true;
                for(const int f : finished) all = all && f != 0;
                if(all) break;
            }
        }
        check_cuda(cudaMemcpyAsync(decoded_ids, t->staged_decoder.data, size_t(B * S_dec) * sizeof(type), cudaMemcpyDeviceToHost, t->stream), "decode: ids D2H");
        check_cuda(cudaStreamSynchronize(t->stream), "decode: ids D2H");
    });
}

// One target position of the cached decoding loop: the decoder side on that position, then the arg-max into the next slot.
static void decode_position(onn_trainer* t, Index i, int end_id)
{
    const Index B = t->micro_batch, S_dec = t->decoder_sequence_length;
    // the output layer leaves logits where it can: softmax and arg-max are one kernel then
    const type* distribution = t->decoder->step(t->decode_ids.data, S_dec, i - 1, true);
    if(t->decoder->output_is_logits())
        check_onn(onn_greedy_next_token_logits(distribution, t->decode_ids.data, reinterpret_cast<int*>(t->decode_finished.data), B, S_dec,
                                               t->vocabulary_size, i, end_id, t->stream), "greedy step");
    else
        check_onn(onn_greedy_next_token_rows(distribution, t->decode_ids.data, reinterpret_cast<int*>(t->decode_finished.data), B, S_dec,
                                             t->vocabulary_size, i, end_id, t->stream), "greedy step");
}

// Replays position i from its graph, capturing it first if need be.  Returns false (nothing has run) if graphs cannot be used.
static bool replay_decode_position(onn_trainer* t, Index i, int end_id)
{
    if(t->decode_graphs.size() < size_t(t->decoder_sequence_length))
    {
        t->decode_graphs.resize(size_t(t->decoder_sequence_length), nullptr);
        t->decode_graph_launches.resize(size_t(t->decoder_sequence_length), 0);
    }
    cudaGraphExec_t& executable = t->decode_graphs[size_t(i)];
    if(!executable)
    {
        const uint64_t launches_before = onn_launch_count();
        cudaGraph_t captured = nullptr;
        bool ok = cudaStreamBeginCapture(t->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if(ok)
        {
            try { decode_position(t, i, end_id); }
            catch(...) { ok = false; }
            ok = (cudaStreamEndCapture(t->stream, &captured) == cudaSuccess) && ok && captured != nullptr;
        }
        if(ok) ok = cudaGraphInstantiate(&executable, captured, 0) == cudaSuccess;
        if(captured) cudaGraphDestroy(captured);
        const uint64_t counted = onn_launch_count() - launches_before;
        onn_launch_count_add(0 - counted);                          // counted at capture, launched below
        if(!ok)
        {
            cudaGetLastError();
            executable = nullptr;
            return false;
        }
        t->decode_graph_launches[size_t(i)] = counted;
    }
    check_cuda(cudaGraphLaunch(executable, t->stream), "decode graph launch");
    onn_launch_count_add(t->decode_graph_launches[size_t(i)]);
    return true;
}

extern "C" int onn_trainer_greedy_decode_cached(onn_trainer* t, const float* encoder_ids, float* decoded_ids, int start_id, int end_id)
{
    if(!t || !encoder_ids || !decoded_ids || t->decoder_only) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        Device::instance().set_compute_stream(t->stream);
        await_parameters(t);
        const Index B = t->micro_batch, S_in = t->input_sequence_length, S_dec = t->decoder_sequence_length;
        if(t->staged_encoder.size() < B * S_in) t->staged_encoder.resize(B * S_in);
        if(t->decode_ids.size() == 0) { t->decode_ids.resize(B * S_dec); t->decode_finished.resize(B); }
        t->decode_finished.fill(0);                                    // read as int

        vector<type> target(size_t(B * S_dec), type(0));
        for(Index b = 0; b < B; b++) target[size_t(b * S_dec)] = type(start_id);
        check_cuda(cudaMemcpyAsync(t->staged_encoder.data, encoder_ids, size_t(B * S_in) * sizeof(type), cudaMemcpyHostToDevice, t->stream), "ids H2D");
        check_cuda(cudaMemcpyAsync(t->decode_ids.data, target.data(), target.size() * sizeof(type), cudaMemcpyHostToDevice, t->stream), "ids H2D");
        check_cuda(cudaStreamSynchronize(t->stream), "decode: ids");

        // encoder side once, through the ordinary forward pass
        BatchCuda batch;
        batch.samples_number = B;
        batch.decoder = TensorViewCuda(t->decode_ids.data, {B, S_dec});
        batch.input = TensorViewCuda(t->staged_encoder.data, {B, S_in});
        vector<char> encoder_side = t->network->layers_depending_on_input(1);
        for(char& flag : encoder_side) flag = !flag;
        t->network->forward_propagate(batch.get_inputs_device(), *t->forward, false, &encoder_side);

        if(!t->decoder) t->decoder = std::make_unique<IncrementalDecoder>(t->network.get(), t->forward.get(), B);
        t->decoder->start();
        // the first call runs eagerly (it configures every kernel); later calls replay one graph per position.  The END id
        // is a captured argument: another one drops the graphs
        bool use_graphs = t->graphs_enabled && t->cached_decodes > 0;
        if(t->decode_end_id != end_id)
            for(cudaGraphExec_t& g : t->decode_graphs) { if(g) cudaGraphExecDestroy(g); g = nullptr; }
        t->decode_end_id = end_id;
        vector<int> finished(size_t(B), 0);
        for(Index i = 1; i < S_dec; i++)
        {
            if(!use_graphs || !replay_decode_position(t, i, end_id))
            {
                use_graphs = false;
                decode_position(t, i, end_id);
            }
            if(i % 8 == 0 || i + 1 == S_dec)
            {
                check_cuda(cudaMemcpyAsync(finished.data(), t->decode_finished.data, size_t(B) * sizeof(int), cudaMemcpyDeviceToHost, t->stream), "decode: flags");
                check_cuda(cudaStreamSynchronize(t->stream), "decode: flags");
                bool all = true;
                for(const int f : finished) all = all && f != 0;
                if(all) break;
            }
        }
        t->cached_decodes++;
        check_cuda(cudaMemcpyAsync(decoded_ids, t->decode_ids.data, size_t(B * S_dec) * sizeof(type), cudaMemcpyDeviceToHost, t->stream), "decode: ids D2H");
        check_cuda(cudaStreamSynchronize(t->stream), "decode: ids D2H");
    });
}

extern "C" int onn_trainer_get_layer_output(onn_trainer* t, int layer, float* host_output, int64_t count)
{
    if(!t || !host_output || layer < 0 || layer >= int(t->network->get_layers_number())) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        const TensorViewCuda outputs = t->forward->layers[size_t(layer)]->outputs;
        if(count > outputs.size()) throw std::runtime_error("get_layer_output: count exceeds the layer's output size");
        check_cuda(cudaStreamSynchronize(t->stream), "synchronize");
        check_cuda(cudaMemcpy(host_output, outputs.data, size_t(count) * sizeof(type), cudaMemcpyDeviceToHost), "get_layer_output");
    });
}

extern "C" int onn_trainer_synchronize(onn_trainer* t)
{
    if(!t) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&] { settle_parameters(t); check_device_status(t); });
}

extern "C" int onn_trainer_exchange_segments(const onn_trainer* t)
{
    return t ? int(t->exchange_graph.segments.size()) : 0;
}

extern "C" int onn_trainer_trace_phases(onn_trainer* t, int enabled)
{
    if(!t) return ONN_ERR_INVALID_ARGUMENT;
    t->trace_phases = enabled != 0;
    t->phases_recorded = false;
    return ONN_OK;
}

extern "C" int onn_trainer_last_step_phases(onn_trainer* t, float* milliseconds3)
{
    if(!t || !milliseconds3) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        if(!t->trace_phases || !t->phases_recorded) throw std::runtime_error("last_step_phases: no traced step (the last micro-batch must have run eagerly)");
        check_cuda(cudaStreamSynchronize(t->stream), "synchronize");
        for(int k = 0; k < 3; k++)
            check_cuda(cudaEventElapsedTime(milliseconds3 + k, t->phase_events[k], t->phase_events[k + 1]), "phase times");
    });
}

extern "C" int onn_trainer_parameters_ready(onn_trainer* t)
{
    if(!t) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&] { await_parameters(t); });
}

extern "C" void* onn_trainer_stream(onn_trainer* t) { return t ? t->stream : nullptr; }
